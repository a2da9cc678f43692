// Expert-parallel exchange overlapped with the grouped GEMM, over peer memory.
//
// Per step every rank (one GPU each)
//   1. plans its routes (ep_route_kernel: destination row of every assignment, origin
//      record beside it, one entry per row bucketed by exchange group) and pushes its
//      token rows straight into the owners' expert-major packed A (ep_dispatch_kernel).
//      Experts are split into a few GROUPS in packed order; the kernel works group by
//      group and, when all of its rows of a group have been written, raises a
//      per-(group, source) flag in every peer's flag array;
//   2. runs ONE grouped GEMM whose tile scheduler holds back the tiles of a group
//      until the flags of all other sources for that group have arrived
//      (GemmParams::gate_*), so the math on early groups overlaps the transfer of
//      late ones;
//   3. sends the result rows back to the rank each row came from, following the
//      per-row origin record the route kernel left beside the row: by default from
//      the epilogue of the GEMM itself (GemmParams::push_*), with ep_return_kernel
//      only raising the "done" flag on every peer afterwards; or, with D kept local,
//      by ep_return_kernel copying the rows after the GEMM;
//   4. waits for the other ranks' "done" flags (ep_wait_flags_kernel).
//
// Kernels of one GPU never wait on one another: rows whose owner is the sending
// rank itself are copied by a launch that precedes the GEMM in the same stream,
// and the GEMM gates on the flags of OTHER ranks only. Every wait is bounded
// (nanosleep polling against a time budget); a wait that runs out records a
// status word the host reads and the kernel carries on.
//
// The reference has no multi-GPU path (its grouped GEMM takes per-expert device
// pointers, baselines/cutlass/cutlass_baseline.cu:243-250); these are the data
// movers either side of that interface for the expert-parallel configuration.
#include <cuda_runtime.h>

#include <cstdint>

#include "bmoe_b200.h"
#include "preload.cuh"
#include "ptx_sm100.cuh"

namespace bmoe {
namespace {

constexpr uint32_t kExThreads = 256;
constexpr uint32_t kExUnroll = 8;          // 16-byte vectors in flight per lane
constexpr uint64_t kOriginRankShift = 40;  // origin record: rank << 40 | assignment

__device__ __forceinline__ void st_release_sys(uint32_t* addr, uint32_t value) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(addr), "r"(value) : "memory");
}

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* addr) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}

__device__ __forceinline__ uint64_t timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ void copy_row(const uint4* __restrict__ s, uint4* __restrict__ d,
                                         uint32_t vec_per_row, uint32_t lane) {
  for (uint32_t v0 = 0; v0 < vec_per_row; v0 += 32 * kExUnroll) {
    uint4 regs[kExUnroll];
#pragma unroll
    for (uint32_t u = 0; u < kExUnroll; ++u) {
      const uint32_t v = v0 + u * 32 + lane;
      if (v < vec_per_row) regs[u] = s[v];
    }
#pragma unroll
    for (uint32_t u = 0; u < kExUnroll; ++u) {
      const uint32_t v = v0 + u * 32 + lane;
      if (v < vec_per_row) d[v] = regs[u];
    }
  }
}

// All CTAs of a launch call this after their last store of a phase: the CTA that
// arrives last raises `value` in slot `slot` of every other rank's flag array.
__device__ __forceinline__ void signal_peers_when_grid_done(uint32_t* counter,
                                                            uint32_t* const* flag_bases,
                                                            uint32_t ranks, uint32_t self,
                                                            uint32_t slot, uint32_t value) {
  __threadfence_system();  // this thread's rows are visible to the peers
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const uint32_t arrived = atomicAdd(counter, 1u);
    if (arrived == gridDim.x - 1) {
      __threadfence_system();
      for (uint32_t r = 0; r < ranks; ++r) {
        if (r != self) st_release_sys(flag_bases[r] + slot, value);
      }
    }
  }
}

// One routed row to copy: token row `token` of this rank's x -> row `row` of rank `to`.
struct RouteEntry {
  uint32_t token;
  uint32_t to;
  uint32_t row;
  uint32_t pad;
};
static_assert(sizeof(RouteEntry) == 16, "one 16-byte load per entry");

struct RouteArgs {
  const int64_t* expert_ids;   // [assignments]
  const int64_t* row_base;     // [experts] first row of (expert, this source) in the owner's A
  const int32_t* owner;        // [experts]
  const uint8_t* group_of;     // [experts] group of the expert on its owner
  uint32_t* cursor;            // [experts] rows handed out so far (zero at step start)
  long long* const* origin_bases;  // [ranks] origin record per packed row
  RouteEntry* entries;         // [assignments] bucketed: groups 0..G-1 (remote), G (local),
                               // G + 1 (rows of copy-engine blocks, into the staging buffer)
  const uint32_t* bucket_offset;   // [groups + 3] from the host's count matrix
  uint32_t* bucket_fill;       // [groups + 2] zero at step start
  const int64_t* staging_row_base;  // [experts] >= 0: copy-engine block, first staging row
  uint64_t staging_rows_cap;
  int32_t* dst_rank_out;       // [assignments] or nullptr: where each assignment went
  int64_t* dst_row_out;        // [assignments] or nullptr
  int32_t* primary_out;        // [assignments] or nullptr: send-once mode (see below)
  uint64_t assignments;
  uint64_t rows_cap;
  uint32_t top_k;
  uint32_t experts;
  uint32_t ranks;
  uint32_t self;
  uint32_t groups;
};

// Send-once mode (primary_out != nullptr): a token routed to several experts of ONE other
// rank crosses NVLink once. Of its assignments to that rank the one with the smallest
// (exchange group, position in the token's top-k list) is the PRIMARY and travels as
// before; the others still get their packed row and origin record, but no route entry:
// primary_out[i] names the primary's assignment and ep_duplicates_kernel tells the owner
// to copy the primary's row (already in its A) into the duplicate's row. -1 = not a
// duplicate.
__device__ __forceinline__ int32_t primary_of(const RouteArgs& a, uint64_t i, int32_t to,
                                              uint32_t group) {
  const uint64_t token = i / a.top_k;
  const uint32_t mine = static_cast<uint32_t>(i - token * a.top_k);
  uint32_t best_group = group, best_j = mine;
  for (uint32_t j = 0; j < a.top_k; ++j) {
    if (j == mine) continue;
    const int64_t e = a.expert_ids[token * a.top_k + j];
    if (e < 0 || e >= static_cast<int64_t>(a.experts) || a.owner[e] != to) continue;
    const uint32_t g = a.group_of[e];
    if (g >= a.groups) continue;
    if (g < best_group || (g == best_group && j < best_j)) {
      best_group = g;
      best_j = j;
    }
  }
  return best_j == mine ? -1 : static_cast<int32_t>(token * a.top_k + best_j);
}

constexpr uint32_t kDuplicateBucket = 0xfffffffeu;   // takes a row, but no route entry

// Route planning, one thread per assignment: destination row from the expert's cursor
// (the order of rows inside an expert changes no result row, only where it sits), the
// origin record beside that row, and one entry in the bucket of the row's exchange
// group (or the local bucket). Lanes that hit the same expert or bucket share one
// atomic. The copy kernels then walk dense lists instead of filtering all assignments
// once per group.
__global__ void __launch_bounds__(256) ep_route_kernel(RouteArgs a) {
  const uint32_t lane = threadIdx.x & 31;
  const uint32_t lanes_below = (1u << lane) - 1u;
  const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
  const uint64_t rounds = (a.assignments + stride - 1) / stride;
  for (uint64_t r = 0; r < rounds; ++r) {  // whole warps stay together for the votes
    const uint64_t i = r * stride + static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    int64_t e = -1;
    int32_t to = -1;
    uint32_t bucket = 0xffffffffu;
    if (i < a.assignments) {
      e = a.expert_ids[i];
      if (e >= 0 && e < static_cast<int64_t>(a.experts)) {
        to = a.owner[e];
        if (to >= 0 && static_cast<uint32_t>(to) < a.ranks) {
          bucket = static_cast<uint32_t>(to) == a.self ? a.groups : a.group_of[e];
          if (bucket > a.groups) bucket = 0xffffffffu;
          // a block that travels as one peer copy is first packed into local staging
          if (bucket < a.groups && a.staging_row_base != nullptr &&
              a.staging_row_base[e] >= 0) {
            bucket = a.groups + 1;
          }
        }
      }
    }
    int32_t primary = -1;
    if (a.primary_out != nullptr && bucket < a.groups) {
      primary = primary_of(a, i, to, bucket);
      if (primary >= 0) bucket = kDuplicateBucket;
    }
    const bool live = bucket != 0xffffffffu;
    const bool has_entry = live && bucket != kDuplicateBucket;
    // one cursor atomic per distinct expert in the warp
    const uint32_t key_e = live ? static_cast<uint32_t>(e) : 0xffffffffu;
    const uint32_t same_e = __match_any_sync(0xffffffffu, key_e);
    uint32_t first_pos = 0;
    const uint32_t lead_e = __ffs(same_e) - 1;
    if (live && lane == lead_e) first_pos = atomicAdd(&a.cursor[e], __popc(same_e));
    first_pos = __shfl_sync(0xffffffffu, first_pos, lead_e);
    // one bucket atomic per distinct bucket in the warp
    const uint32_t same_b = __match_any_sync(0xffffffffu, bucket);
    uint32_t first_slot = 0;
    const uint32_t lead_b = __ffs(same_b) - 1;
    if (has_entry && lane == lead_b) {
      first_slot = atomicAdd(&a.bucket_fill[bucket], __popc(same_b));
    }
    first_slot = __shfl_sync(0xffffffffu, first_slot, lead_b);
    if (!live) {
      if (a.primary_out != nullptr && i < a.assignments) a.primary_out[i] = -1;
      continue;
    }
    const int64_t row = a.row_base[e] + first_pos + __popc(same_e & lanes_below);
    if (!has_entry) {
      // a duplicate: its row and origin record, no entry; the owner fills the row itself
      const bool fits = row >= 0 && static_cast<uint64_t>(row) < a.rows_cap;
      if (fits) {
        a.origin_bases[to][row] =
            static_cast<long long>((static_cast<uint64_t>(a.self) << kOriginRankShift) | i);
      }
      a.primary_out[i] = fits ? primary : -1;
      if (a.dst_rank_out != nullptr) a.dst_rank_out[i] = to;
      if (a.dst_row_out != nullptr) a.dst_row_out[i] = fits ? row : -1;
      continue;
    }
    if (a.primary_out != nullptr) a.primary_out[i] = -1;
    const uint32_t slot = a.bucket_offset[bucket] + first_slot + __popc(same_b & lanes_below);
    if (slot >= a.bucket_offset[bucket + 1] || slot >= a.assignments) {
      if (a.dst_row_out != nullptr) a.dst_row_out[i] = -1;   // nothing was sent for it
      continue;
    }
    // A bad table must never become a stray access to another GPU's memory: the slot
    // this assignment reserved gets an entry no rank owns (the copy kernels skip it)
    // instead of keeping whatever an earlier step left there.
    if (row < 0 || static_cast<uint64_t>(row) >= a.rows_cap) {
      RouteEntry none;
      none.token = 0xffffffffu;
      none.to = 0xffffffffu;
      none.row = 0xffffffffu;
      none.pad = 0;
      a.entries[slot] = none;
      if (a.dst_row_out != nullptr) a.dst_row_out[i] = -1;
      continue;
    }
    a.origin_bases[to][row] =
        static_cast<long long>((static_cast<uint64_t>(a.self) << kOriginRankShift) | i);
    RouteEntry entry;
    entry.token = static_cast<uint32_t>(i / a.top_k);
    entry.to = static_cast<uint32_t>(to);
    entry.row = static_cast<uint32_t>(row);
    entry.pad = 0;
    if (bucket == a.groups + 1) {
      // staged row: same position inside the block as in the owner's A
      const int64_t staged = a.staging_row_base[e] + (row - a.row_base[e]);
      entry.to = a.self;
      entry.row = static_cast<uint32_t>(staged);
      if (staged < 0 || static_cast<uint64_t>(staged) >= a.staging_rows_cap) {
        entry.token = 0xffffffffu;
        entry.to = 0xffffffffu;   // no rank owns it: the copy kernels skip the entry
      }
    }
    a.entries[slot] = entry;
    if (a.dst_rank_out != nullptr) a.dst_rank_out[i] = to;
    if (a.dst_row_out != nullptr) a.dst_row_out[i] = row;
  }
}

// Send-once mode, second pass: one record {row of the primary, row of the duplicate} per
// duplicate assignment, appended to the list of (exchange group of the duplicate, this
// source) in the OWNER's memory; when the whole grid is done the last CTA publishes the list
// lengths there. The owner's GEMM kernel copies primary -> duplicate once this source's
// flag for the group is up (the primary belongs to the same or an earlier group of the same
// source, so it has landed by then). Runs after ep_route_kernel and before the launch that
// pushes the rows and raises the flags, in one stream.
struct DuplicateArgs {
  const int64_t* expert_ids;     // [assignments]
  const int32_t* owner;          // [experts]
  const uint8_t* group_of;       // [experts]
  const int32_t* primary;        // [assignments] from ep_route_kernel
  const int64_t* row_of;         // [assignments] packed row of every assignment (-1: none)
  uint2* const* record_bases;    // [ranks] record lists: [groups][ranks][record_cap]
  uint32_t* const* count_bases;  // [ranks] list lengths: [groups][ranks]
  uint32_t* fill;                // [ranks][groups] zero at step start
  uint32_t* done_counter;        // zero at step start
  uint64_t assignments;
  uint32_t record_cap;
  uint32_t experts;
  uint32_t ranks;
  uint32_t self;
  uint32_t groups;
};

__global__ void __launch_bounds__(256) ep_duplicates_kernel(DuplicateArgs a) {
  const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
  for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < a.assignments;
       i += stride) {
    const int32_t first = a.primary[i];
    if (first < 0 || static_cast<uint64_t>(first) >= a.assignments) continue;
    const int64_t e = a.expert_ids[i];
    if (e < 0 || e >= static_cast<int64_t>(a.experts)) continue;
    const int32_t to = a.owner[e];
    const uint32_t g = a.group_of[e];
    const int64_t from_row = a.row_of[first], to_row = a.row_of[i];
    if (to < 0 || static_cast<uint32_t>(to) >= a.ranks || static_cast<uint32_t>(to) == a.self ||
        g >= a.groups || from_row < 0 || to_row < 0) {
      continue;
    }
    const uint32_t at = atomicAdd(&a.fill[static_cast<uint32_t>(to) * a.groups + g], 1u);
    if (at >= a.record_cap) continue;   // cannot happen with record_cap >= assignments
    a.record_bases[to][(static_cast<size_t>(g) * a.ranks + a.self) * a.record_cap + at] =
        make_uint2(static_cast<uint32_t>(from_row), static_cast<uint32_t>(to_row));
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint32_t arrived = atomicAdd(a.done_counter, 1u);
    if (arrived == gridDim.x - 1) {
      __threadfence_system();
      for (uint32_t r = 0; r < a.ranks; ++r) {
        if (r == a.self) continue;
        for (uint32_t g = 0; g < a.groups; ++g) {
          const uint32_t n = a.fill[r * a.groups + g];
          a.count_bases[r][g * a.ranks + a.self] = n < a.record_cap ? n : a.record_cap;
        }
      }
      __threadfence_system();
    }
  }
}

struct DispatchArgs {
  const uint4* x;              // [tokens, k] BF16 token rows of this rank
  const RouteEntry* entries;   // bucketed route entries (ep_route_kernel)
  const uint32_t* bucket_offset;   // [groups + 2]
  uint4* const* a_bases;       // [ranks] packed A of every rank
  uint32_t* const* flag_bases; // [ranks] flag arrays
  uint32_t* group_done;        // [groups] CTA arrival counters (zero at step start)
  uint32_t* chunk_next;        // [groups + 1] next unclaimed entry per bucket (zero at start)
  uint64_t tokens;
  uint64_t rows_cap;
  uint32_t vec_per_row;
  uint32_t ranks;
  uint32_t self;
  uint32_t groups;
  uint32_t mode;               // BMOE_EP_LOCAL / BMOE_EP_REMOTE / BMOE_EP_ALL
  uint32_t epoch;
  uint32_t span;               // entries per claim: 1..32
  uint32_t row_bytes;
  uint32_t* status;            // optional: set when a bulk-copy wait ran out
  const uint32_t* bucket_fill; // optional [groups + 2]: entries really written per bucket
                               // (send-once mode leaves gaps at the end of a bucket)
};

// Bucket by bucket (exchange groups in order, then - or only - the local bucket), a
// warp claims `span` entries at a time from a shared counter (SMs that also push rows
// over NVLink or run GEMM CTAs are slower, so a static split would wait for them) and
// copies those token rows one after the other, 512 contiguous bytes per instruction.
// When every CTA has finished a remote group, the last one raises the group's flag on
// all peers.
__global__ void __launch_bounds__(1024) ep_dispatch_kernel(DispatchArgs a) {
  const uint32_t lane = threadIdx.x & 31;
  const uint32_t span = a.span;
  const uint32_t first_bucket = a.mode == BMOE_EP_LOCAL  ? a.groups
                                : a.mode == BMOE_EP_PACK ? a.groups + 1u
                                                         : 0u;
  const uint32_t end_bucket = a.mode == BMOE_EP_REMOTE ? a.groups
                              : a.mode == BMOE_EP_PACK ? a.groups + 2u
                                                       : a.groups + 1u;
  for (uint32_t b = first_bucket; b < end_bucket; ++b) {
    const uint32_t begin = a.bucket_offset[b];
    uint32_t count = a.bucket_offset[b + 1] - begin;
    if (a.bucket_fill != nullptr && a.bucket_fill[b] < count) count = a.bucket_fill[b];
    while (true) {
      uint32_t at = 0;
      if (lane == 0) at = atomicAdd(&a.chunk_next[b], span);
      at = __shfl_sync(0xffffffffu, at, 0);
      if (at >= count) break;
      RouteEntry entry{};
      bool have = false;
      if (lane < span && at + lane < count) {
        entry = a.entries[begin + at + lane];
        // entries come from this GPU's own route kernel; check them all the same
        have = entry.to < a.ranks && entry.row < a.rows_cap && entry.token < a.tokens;
      }
      uint32_t todo = __ballot_sync(0xffffffffu, have);
      while (todo != 0) {
        const uint32_t l = __ffs(todo) - 1;
        todo &= todo - 1;
        const uint32_t token = __shfl_sync(0xffffffffu, entry.token, l);
        const uint32_t to = __shfl_sync(0xffffffffu, entry.to, l);
        const uint32_t row = __shfl_sync(0xffffffffu, entry.row, l);
        copy_row(a.x + static_cast<uint64_t>(token) * a.vec_per_row,
                 a.a_bases[to] + static_cast<uint64_t>(row) * a.vec_per_row, a.vec_per_row, lane);
      }
    }
    if (b < a.groups && a.ranks > 1) {
      signal_peers_when_grid_done(&a.group_done[b], a.flag_bases, a.ranks, a.self,
                                  b * a.ranks + a.self, a.epoch);
    }
  }
}

// Same walk as ep_dispatch_kernel, but the rows travel through the TMA engine: every
// warp owns one row-sized stage in shared memory; its first lane loads a token row with
// one bulk copy (global -> shared, counted on an mbarrier) and sends it on with one bulk
// copy (shared -> peer memory). No load/store unit of the SM waits for NVLink. Needs
// SMs of its own (the stages take most of the shared memory). Waits are bounded; a wait
// that runs out sets *status and the warp stops copying (the flags are still raised so
// that no other rank is left waiting for them; the status word tells the host).
constexpr uint32_t kBulkMaxWarps = 16;   // stages per CTA: as many rows as fit in shared memory

__global__ void __launch_bounds__(kBulkMaxWarps * 32) ep_dispatch_bulk_kernel(DispatchArgs a) {
  extern __shared__ __align__(128) uint8_t bulk_smem[];
  const uint32_t lane = threadIdx.x & 31;
  const uint32_t warp = threadIdx.x >> 5;
  const uint32_t stage_bytes = (a.row_bytes + 127u) & ~127u;
  const uint32_t smem0 = ptx::smem_addr(bulk_smem);
  const uint32_t warps = blockDim.x >> 5;
  const uint32_t stage = smem0 + warp * stage_bytes;
  const uint32_t bar = smem0 + warps * stage_bytes + warp * 8;
  volatile uint32_t* const abort_word = reinterpret_cast<volatile uint32_t*>(
      bulk_smem + warps * stage_bytes + warps * 8 + warp * 4);
  if (lane == 0) {
    ptx::mbar_init(bar, 1);
    *abort_word = 0;
    ptx::fence_barrier_init();
  }
  __syncwarp();
  uint32_t parity = 0;
  bool alive = true;
  const uint32_t span = a.span;
  const uint32_t first_bucket = a.mode == BMOE_EP_LOCAL ? a.groups : 0u;
  const uint32_t end_bucket = a.mode == BMOE_EP_REMOTE ? a.groups : a.groups + 1u;
  const uint8_t* const x = reinterpret_cast<const uint8_t*>(a.x);
  for (uint32_t b = first_bucket; b < end_bucket; ++b) {
    const uint32_t begin = a.bucket_offset[b];
    uint32_t count = a.bucket_offset[b + 1] - begin;
    if (a.bucket_fill != nullptr && a.bucket_fill[b] < count) count = a.bucket_fill[b];
    while (alive) {
      uint32_t at = 0;
      if (lane == 0) at = atomicAdd(&a.chunk_next[b], span);
      at = __shfl_sync(0xffffffffu, at, 0);
      if (at >= count) break;
      RouteEntry entry{};
      bool have = false;
      if (lane < span && at + lane < count) {
        entry = a.entries[begin + at + lane];
        have = entry.to < a.ranks && entry.row < a.rows_cap && entry.token < a.tokens;
      }
      uint32_t todo = __ballot_sync(0xffffffffu, have);
      while (todo != 0 && alive) {
        const uint32_t l = __ffs(todo) - 1;
        todo &= todo - 1;
        const uint32_t token = __shfl_sync(0xffffffffu, entry.token, l);
        const uint32_t to = __shfl_sync(0xffffffffu, entry.to, l);
        const uint32_t row = __shfl_sync(0xffffffffu, entry.row, l);
        if (lane == 0) {
          ptx::tma_store_wait_read<0>();   // the previous row has left the stage
          ptx::mbar_arrive_expect_tx(bar, a.row_bytes);
          ptx::bulk_load_1d(stage, x + static_cast<uint64_t>(token) * a.row_bytes, a.row_bytes, bar);
          if (ptx::mbar_wait(bar, parity, abort_word, 1000000000ull)) {
            ptx::bulk_store_1d(reinterpret_cast<uint8_t*>(a.a_bases[to]) +
                                   static_cast<uint64_t>(row) * a.row_bytes,
                               stage, a.row_bytes);
            ptx::tma_store_commit();
          } else if (a.status != nullptr) {
            atomicCAS(a.status, 0u, 0x40000000u | b);
          }
        }
        parity ^= 1u;
        alive = __shfl_sync(0xffffffffu, *abort_word == 0 ? 1u : 0u, 0) != 0;
      }
    }
    if (lane == 0) {
      ptx::tma_store_wait_all();  // this warp's rows of the bucket have landed
      ptx::fence_proxy_async_all();
      if (!alive) {
        // a load that was given up on may still be writing the stage: let it land
        const uint64_t t0 = timer_ns();
        while (timer_ns() - t0 < 200000) __nanosleep(1000);
      }
    }
    __syncwarp();
    if (b < a.groups && a.ranks > 1) {
      signal_peers_when_grid_done(&a.group_done[b], a.flag_bases, a.ranks, a.self,
                                  b * a.ranks + a.self, a.epoch);
    }
  }
}

struct ReturnArgs {
  const uint4* d;              // [rows, n] BF16 packed results of this rank
  const long long* origin;     // [rows] origin record of every packed row
  uint4* const* y_bases;       // [ranks] result buffers in assignment order
  uint32_t* const* flag_bases;
  uint32_t* done_counter;      // CTA arrival counter (zero at step start)
  uint64_t rows;
  uint64_t y_rows_cap;
  uint32_t vec_per_row;
  uint32_t ranks;
  uint32_t self;
  uint32_t flag_slot;          // slot of this rank's "done" flag in the peers' arrays
  uint32_t epoch;
};

__global__ void __launch_bounds__(kExThreads) ep_return_kernel(ReturnArgs a) {
  const uint32_t lane = threadIdx.x & 31;
  const uint64_t warps = static_cast<uint64_t>(gridDim.x) * (kExThreads / 32);
  for (uint64_t r = static_cast<uint64_t>(blockIdx.x) * (kExThreads / 32) + (threadIdx.x >> 5);
       r < a.rows; r += warps) {
    const uint64_t rec = static_cast<uint64_t>(a.origin[r]);
    const uint64_t to = rec >> kOriginRankShift;
    const uint64_t at = rec & ((1ull << kOriginRankShift) - 1);
    if (to >= a.ranks || at >= a.y_rows_cap) continue;
    copy_row(a.d + r * a.vec_per_row, a.y_bases[to] + at * a.vec_per_row, a.vec_per_row, lane);
  }
  if (a.ranks > 1) {
    signal_peers_when_grid_done(a.done_counter, a.flag_bases, a.ranks, a.self, a.flag_slot,
                                a.epoch);
  }
}

// One warp; lane r watches slot first_slot + r (r != self) until it reaches
// `epoch`. Gives up after budget_ns and records which rank was missing.
__global__ void ep_wait_flags_kernel(const uint32_t* flags, uint32_t first_slot, uint32_t ranks,
                                     uint32_t self, uint32_t epoch, uint64_t budget_ns,
                                     uint32_t* status) {
  const uint32_t r = threadIdx.x;
  if (r >= ranks || r == self) return;
  const uint32_t* flag = flags + first_slot + r;
  uint64_t start = 0;
  for (uint32_t spin = 1;; ++spin) {
    if (static_cast<int32_t>(ld_acquire_sys(flag) - epoch) >= 0) return;
    if ((spin & 0xf) == 0) {
      const uint64_t now = timer_ns();
      if (start == 0) {
        start = now;
      } else if (now - start > budget_ns) {
        if (status != nullptr) {
          atomicCAS(status, 0u, 0x80000000u | (first_slot << 8) | r);
        }
        return;
      }
    }
    __nanosleep(200);
  }
}

// Routed rows per expert of this rank, and (optionally) the expert -> shard mapping of
// split experts, in one pass: counts[id] += 1 for every valid assignment, where id is
// the expert, or shard_base[expert] + i % parts[expert] when shards are given (the
// shard ids are also written to ids_out). Invalid expert ids count nowhere and map to
// -1. Shared-memory histogram per CTA, flushed with one atomic per non-empty bin.
constexpr uint32_t kCountBins = 4096;

__global__ void __launch_bounds__(256)
ep_count_kernel(const int64_t* __restrict__ expert_ids, uint64_t assignments, uint32_t experts,
                const int64_t* __restrict__ parts, const int64_t* __restrict__ shard_base,
                uint32_t bins, int64_t* __restrict__ ids_out,
                unsigned long long* __restrict__ counts) {
  __shared__ uint32_t hist[kCountBins];
  for (uint32_t b = threadIdx.x; b < bins; b += blockDim.x) hist[b] = 0;
  __syncthreads();
  const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
  for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < assignments;
       i += stride) {
    const int64_t e = expert_ids[i];
    int64_t id = -1;
    if (e >= 0 && e < static_cast<int64_t>(experts)) {
      id = e;
      if (parts != nullptr) {
        const int64_t p = parts[e];
        id = p > 0 ? shard_base[e] + static_cast<int64_t>(i % static_cast<uint64_t>(p)) : -1;
      }
      if (id < 0 || id >= static_cast<int64_t>(bins)) id = -1;
    }
    if (ids_out != nullptr) ids_out[i] = id;
    if (id >= 0) atomicAdd(&hist[id], 1u);
  }
  __syncthreads();
  for (uint32_t b = threadIdx.x; b < bins; b += blockDim.x) {
    if (hist[b] != 0) atomicAdd(&counts[b], static_cast<unsigned long long>(hist[b]));
  }
}

// ---------------------------------------------------------------------------
// Step tables on the device (what the Python layer's host planner computes with numpy).
// One CTA; position i runs over the experts sorted by (owner, id), so an owner's experts
// are one contiguous segment in packed order.
// ---------------------------------------------------------------------------
struct PlanArgs {
  const int64_t* counts_all;
  const int32_t* owner;
  const int32_t* order;
  int64_t* row_base;
  uint8_t* group_of;
  uint8_t* group_local;
  uint32_t* expert_row;
  uint32_t* local_rows;
  uint32_t* bucket_offset;
  uint32_t* totals;
  uint64_t rows_cap;
  uint32_t experts;
  uint32_t ranks;
  uint32_t self;
  uint32_t groups;
  uint32_t tile_m;
};

constexpr uint32_t kPlanThreads = 1024;
constexpr uint32_t kPlanMaxExperts = 4096;
constexpr uint32_t kPlanMaxRanks = 32;
constexpr uint32_t kTileShift = 40;   // scanned value: rows | tiles << 40

__global__ void __launch_bounds__(kPlanThreads) ep_plan_kernel(PlanArgs a) {
  extern __shared__ unsigned long long plan_scan[];   // [experts] exclusive (rows | tiles << 40)
  __shared__ unsigned long long warp_sum[kPlanThreads / 32];
  __shared__ uint32_t seg_first[kPlanMaxRanks + 1];   // first position of every owner's segment
  __shared__ unsigned long long bucket[BMOE_EP_MAX_GROUPS + 2];
  const uint32_t tid = threadIdx.x;
  const uint32_t lane = tid & 31, warp = tid >> 5;
  const uint32_t per_thread = (a.experts + kPlanThreads - 1) / kPlanThreads;   // <= 4
  const uint32_t first = tid * per_thread;
  for (uint32_t r = tid; r <= kPlanMaxRanks; r += kPlanThreads) seg_first[r] = a.experts;
  for (uint32_t b = tid; b < BMOE_EP_MAX_GROUPS + 2; b += kPlanThreads) bucket[b] = 0;
  __syncthreads();

  // totals per expert (in packed order), and where each owner's segment starts
  unsigned long long value[4];
  unsigned long long mine = 0;
  for (uint32_t j = 0; j < per_thread; ++j) {
    const uint32_t i = first + j;
    value[j] = 0;
    if (i >= a.experts) continue;
    const int32_t e = a.order[i];
    unsigned long long rows = 0;
    for (uint32_t r = 0; r < a.ranks; ++r) {
      rows += static_cast<unsigned long long>(a.counts_all[static_cast<size_t>(r) * a.experts + e]);
    }
    const unsigned long long tiles = (rows + a.tile_m - 1) / a.tile_m;
    value[j] = rows | (tiles << kTileShift);
    mine += value[j];
    const int32_t o = a.owner[e];
    if ((i == 0 || a.owner[a.order[i - 1]] != o) && o >= 0 &&
        static_cast<uint32_t>(o) < a.ranks) {
      seg_first[o] = i;
    }
  }
  // block-wide exclusive scan of the per-thread sums
  unsigned long long inclusive = mine;
  for (uint32_t d = 1; d < 32; d <<= 1) {
    const unsigned long long up = __shfl_up_sync(0xffffffffu, inclusive, d);
    if (lane >= d) inclusive += up;
  }
  if (lane == 31) warp_sum[warp] = inclusive;
  __syncthreads();
  if (warp == 0) {
    unsigned long long w = warp_sum[lane];
    for (uint32_t d = 1; d < 32; d <<= 1) {
      const unsigned long long up = __shfl_up_sync(0xffffffffu, w, d);
      if (lane >= d) w += up;
    }
    warp_sum[lane] = w;   // inclusive over warps
  }
  __syncthreads();
  unsigned long long running = inclusive - mine + (warp == 0 ? 0ull : warp_sum[warp - 1]);
  for (uint32_t j = 0; j < per_thread; ++j) {
    const uint32_t i = first + j;
    if (i < a.experts) plan_scan[i] = running;
    running += value[j];
  }
  const unsigned long long grand = warp_sum[kPlanThreads / 32 - 1];
  __syncthreads();
  // an owner without experts starts where the next one does
  if (tid == 0) {
    seg_first[a.ranks] = a.experts;
    for (int32_t r = static_cast<int32_t>(a.ranks) - 1; r >= 0; --r) {
      if (seg_first[r] > seg_first[r + 1]) seg_first[r] = seg_first[r + 1];
    }
  }
  __syncthreads();

  const unsigned long long row_mask = (1ull << kTileShift) - 1;
  const uint32_t local_first = seg_first[a.self];
  for (uint32_t j = 0; j < per_thread; ++j) {
    const uint32_t i = first + j;
    if (i >= a.experts) continue;
    const int32_t e = a.order[i];
    const uint32_t o = static_cast<uint32_t>(a.owner[e]);
    if (o >= a.ranks) continue;   // an expert nobody owns takes part in nothing
    const uint32_t s0 = seg_first[o], s1 = seg_first[o + 1];
    const unsigned long long at = plan_scan[i], seg = plan_scan[s0];
    const unsigned long long seg_end = s1 < a.experts ? plan_scan[s1] : grand;
    unsigned long long before_me = 0, from_me = 0;
    for (uint32_t r = 0; r <= a.self; ++r) {
      const unsigned long long c =
          static_cast<unsigned long long>(a.counts_all[static_cast<size_t>(r) * a.experts + e]);
      if (r < a.self) before_me += c; else from_me = c;
    }
    const unsigned long long row_in_owner = (at & row_mask) - (seg & row_mask);
    a.row_base[e] = static_cast<int64_t>(row_in_owner + before_me);
    uint32_t group = 0;
    if (a.groups > 1) {
      const unsigned long long tiles_before = (at >> kTileShift) - (seg >> kTileShift);
      unsigned long long owner_tiles = (seg_end >> kTileShift) - (seg >> kTileShift);
      if (owner_tiles == 0) owner_tiles = 1;
      const unsigned long long g = tiles_before * a.groups / owner_tiles;
      group = g < a.groups - 1 ? static_cast<uint32_t>(g) : a.groups - 1;
    }
    a.group_of[e] = static_cast<uint8_t>(group);
    if (o == a.self) {
      const uint32_t local = i - local_first;
      a.group_local[local] = static_cast<uint8_t>(group);
      a.expert_row[local] = static_cast<uint32_t>(row_in_owner);
      a.local_rows[local] = static_cast<uint32_t>(value[j] & row_mask);
      if (from_me != 0) atomicAdd(&bucket[a.groups], from_me);
    } else if (from_me != 0) {
      atomicAdd(&bucket[group], from_me);
    }
  }
  __syncthreads();
  if (tid == 0) {
    uint32_t at = 0;
    for (uint32_t b = 0; b < a.groups + 2; ++b) {
      a.bucket_offset[b] = at;
      at += static_cast<uint32_t>(bucket[b]);   // bucket groups + 1 (peer copies) stays empty
    }
    a.bucket_offset[a.groups + 2] = at;
    const uint32_t l1 = seg_first[a.self + 1];
    const unsigned long long owned =
        ((l1 < a.experts ? plan_scan[l1] : grand) & row_mask) -
        ((local_first < a.experts ? plan_scan[local_first] : grand) & row_mask);
    a.totals[0] = static_cast<uint32_t>(owned < 0xffffffffull ? owned : 0xffffffffull);
    a.totals[1] = owned > a.rows_cap ? 1u : 0u;
  }
}

uint32_t device_sms() {
  int device = 0, sms = 0;
  if (cudaGetDevice(&device) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess ||
      sms <= 0) {
    return 148;
  }
  return static_cast<uint32_t>(sms);
}

}  // namespace
}  // namespace bmoe

extern "C" int bmoe_ep_count(const int64_t* expert_ids_dev, uint64_t assignments,
                             uint32_t experts, const int64_t* parts_dev,
                             const int64_t* shard_base_dev, uint32_t bins, int64_t* ids_out_dev,
                             int64_t* counts_dev, void* stream) {
  if (counts_dev == nullptr || bins == 0 || bins > bmoe::kCountBins || experts == 0 ||
      (assignments != 0 && expert_ids_dev == nullptr) ||
      ((parts_dev == nullptr) != (shard_base_dev == nullptr)) ||
      (parts_dev == nullptr && bins != experts)) {
    return BMOE_INVALID_ARGUMENT;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (cudaMemsetAsync(counts_dev, 0, sizeof(int64_t) * bins, s) != cudaSuccess) {
    return BMOE_CUDA_ERROR;
  }
  if (assignments == 0) return BMOE_OK;
  const uint64_t want = (assignments + 1023) / 1024;   // four assignments per thread
  const uint64_t cap = 2ull * bmoe::device_sms();
  const uint32_t grid = static_cast<uint32_t>(want < cap ? want : cap);
  bmoe::ep_count_kernel<<<grid, 256, 0, s>>>(
      expert_ids_dev, assignments, experts, parts_dev, shard_base_dev, bins, ids_out_dev,
      reinterpret_cast<unsigned long long*>(counts_dev));
  return cudaPeekAtLastError() == cudaSuccess ? BMOE_OK : BMOE_CUDA_ERROR;
}

extern "C" int bmoe_ep_plan(const bmoe_ep_plan_args* args) {
  if (args == nullptr) return BMOE_INVALID_ARGUMENT;
  const bmoe_ep_plan_args& c = *args;
  if (c.experts == 0 || c.experts > bmoe::kPlanMaxExperts || c.ranks == 0 ||
      c.ranks > bmoe::kPlanMaxRanks || c.self >= c.ranks || c.groups == 0 ||
      c.groups > BMOE_EP_MAX_GROUPS || c.tile_m == 0 || c.counts_all_dev == nullptr ||
      c.owner_dev == nullptr || c.order_dev == nullptr || c.row_base_dev == nullptr ||
      c.group_of_dev == nullptr || c.group_local_dev == nullptr || c.expert_row_dev == nullptr ||
      c.local_rows_dev == nullptr || c.bucket_offset_dev == nullptr || c.totals_dev == nullptr) {
    return BMOE_INVALID_ARGUMENT;
  }
  bmoe::PlanArgs a;
  a.counts_all = c.counts_all_dev;
  a.owner = c.owner_dev;
  a.order = c.order_dev;
  a.row_base = c.row_base_dev;
  a.group_of = c.group_of_dev;
  a.group_local = c.group_local_dev;
  a.expert_row = c.expert_row_dev;
  a.local_rows = c.local_rows_dev;
  a.bucket_offset = c.bucket_offset_dev;
  a.totals = c.totals_dev;
  a.rows_cap = c.rows_cap;
  a.experts = c.experts;
  a.ranks = c.ranks;
  a.self = c.self;
  a.groups = c.groups;
  a.tile_m = c.tile_m;
  bmoe::ep_plan_kernel<<<1, bmoe::kPlanThreads, sizeof(unsigned long long) * c.experts,
                         static_cast<cudaStream_t>(c.stream)>>>(a);
  return cudaPeekAtLastError() == cudaSuccess ? BMOE_OK : BMOE_CUDA_ERROR;
}

extern "C" int bmoe_ep_route(const bmoe_ep_route_args* args) {
  if (args == nullptr) return BMOE_INVALID_ARGUMENT;
  const bmoe_ep_route_args& c = *args;
  if (c.ranks == 0 || c.self >= c.ranks || c.groups == 0 || c.groups > BMOE_EP_MAX_GROUPS ||
      c.top_k == 0 || c.assignments > 0xffffffffull || c.rows_cap > 0xffffffffull ||
      c.row_base_dev == nullptr || c.owner_dev == nullptr || c.group_of_dev == nullptr ||
      c.cursor_dev == nullptr || c.origin_bases_dev == nullptr || c.entries_dev == nullptr ||
      c.bucket_offset_dev == nullptr || c.bucket_fill_dev == nullptr ||
      (c.assignments != 0 && c.expert_ids_dev == nullptr)) {
    return BMOE_INVALID_ARGUMENT;
  }
  if (c.assignments == 0) return BMOE_OK;
  bmoe::RouteArgs a;
  a.expert_ids = c.expert_ids_dev;
  a.row_base = c.row_base_dev;
  a.owner = c.owner_dev;
  a.group_of = c.group_of_dev;
  a.cursor = c.cursor_dev;
  a.origin_bases = reinterpret_cast<long long* const*>(c.origin_bases_dev);
  a.entries = static_cast<bmoe::RouteEntry*>(c.entries_dev);
  a.bucket_offset = c.bucket_offset_dev;
  a.bucket_fill = c.bucket_fill_dev;
  a.dst_rank_out = c.dst_rank_out_dev;
  a.dst_row_out = c.dst_row_out_dev;
  a.assignments = c.assignments;
  a.rows_cap = c.rows_cap;
  a.top_k = c.top_k;
  a.experts = c.experts;
  a.ranks = c.ranks;
  a.self = c.self;
  a.groups = c.groups;
  a.staging_row_base = c.staging_row_base_dev;
  a.staging_rows_cap = c.staging_rows_cap;
  a.primary_out = c.primary_out_dev;
  if (c.primary_out_dev != nullptr &&
      (c.dst_row_out_dev == nullptr || c.staging_row_base_dev != nullptr)) {
    return BMOE_INVALID_ARGUMENT;   // send-once needs the row of every assignment
  }
  const uint64_t want = (c.assignments + 255) / 256;
  const uint64_t cap = 4ull * bmoe::device_sms();
  const uint32_t grid = static_cast<uint32_t>(want < cap ? want : cap);
  bmoe::ep_route_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(c.stream)>>>(a);
  return cudaPeekAtLastError() == cudaSuccess ? BMOE_OK : BMOE_CUDA_ERROR;
}

extern "C" int bmoe_ep_duplicates(const bmoe_ep_duplicates_args* args) {
  if (args == nullptr) return BMOE_INVALID_ARGUMENT;
  const bmoe_ep_duplicates_args& c = *args;
  if (c.ranks == 0 || c.self >= c.ranks || c.groups == 0 || c.groups > BMOE_EP_MAX_GROUPS ||
      c.record_cap == 0 || c.owner_dev == nullptr || c.group_of_dev == nullptr ||
      c.primary_dev == nullptr || c.row_of_dev == nullptr || c.record_bases_dev == nullptr ||
      c.count_bases_dev == nullptr || c.fill_dev == nullptr || c.done_counter_dev == nullptr ||
      (c.assignments != 0 && c.expert_ids_dev == nullptr)) {
    return BMOE_INVALID_ARGUMENT;
  }
  bmoe::DuplicateArgs a;
  a.expert_ids = c.expert_ids_dev;
  a.owner = c.owner_dev;
  a.group_of = c.group_of_dev;
  a.primary = c.primary_dev;
  a.row_of = c.row_of_dev;
  a.record_bases = reinterpret_cast<uint2* const*>(c.record_bases_dev);
  a.count_bases = reinterpret_cast<uint32_t* const*>(c.count_bases_dev);
  a.fill = c.fill_dev;
  a.done_counter = c.done_counter_dev;
  a.assignments = c.assignments;
  a.record_cap = c.record_cap;
  a.experts = c.experts;
  a.ranks = c.ranks;
  a.self = c.self;
  a.groups = c.groups;
  const uint64_t want = (c.assignments + 255) / 256;
  const uint64_t cap = 2ull * bmoe::device_sms();
  uint32_t grid = static_cast<uint32_t>(want < cap ? want : cap);
  if (grid == 0) grid = 1;   // the list lengths are published even when there is nothing
  bmoe::ep_duplicates_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(c.stream)>>>(a);
  return cudaPeekAtLastError() == cudaSuccess ? BMOE_OK : BMOE_CUDA_ERROR;
}

extern "C" int bmoe_ep_dispatch(const bmoe_ep_dispatch_args* args) {
  if (args == nullptr) return BMOE_INVALID_ARGUMENT;
  const bmoe_ep_dispatch_args& c = *args;
  if (c.ranks == 0 || c.self >= c.ranks || c.groups == 0 || c.groups > BMOE_EP_MAX_GROUPS ||
      c.mode > BMOE_EP_PACK || c.row_bytes == 0 || c.row_bytes % 16 != 0 ||
      (c.mode == BMOE_EP_PACK && c.bulk_copies != 0) ||
      c.a_bases_dev == nullptr || c.entries_dev == nullptr || c.bucket_offset_dev == nullptr ||
      c.chunk_next_dev == nullptr || (c.assignments != 0 && c.x_dev == nullptr) ||
      (c.ranks > 1 && (c.mode == BMOE_EP_REMOTE || c.mode == BMOE_EP_ALL) &&
       (c.flag_bases_dev == nullptr || c.group_done_dev == nullptr))) {
    return BMOE_INVALID_ARGUMENT;
  }
  bmoe::DispatchArgs a;
  a.x = static_cast<const uint4*>(c.x_dev);
  a.entries = static_cast<const bmoe::RouteEntry*>(c.entries_dev);
  a.bucket_offset = c.bucket_offset_dev;
  a.a_bases = reinterpret_cast<uint4* const*>(c.a_bases_dev);
  a.flag_bases = reinterpret_cast<uint32_t* const*>(c.flag_bases_dev);
  a.group_done = c.group_done_dev;
  a.chunk_next = c.chunk_next_dev;
  a.tokens = c.tokens;
  a.rows_cap = c.rows_cap;
  a.vec_per_row = c.row_bytes / 16;
  a.ranks = c.ranks;
  a.self = c.self;
  a.groups = c.groups;
  a.mode = c.mode;
  a.epoch = c.epoch;
  // Remote rows, default shape: 256-thread CTAs on fewer than half of the SMs. Each
  // fits beside a resident GEMM CTA, so the copy runs while the GEMM computes, but an
  // SM whose stores wait for NVLink slows everything else on it (measured: 64 CTAs
  // move the rows as fast as 148 and disturb the GEMM much less). Callers that keep
  // some SMs free of GEMM CTAs ask for a few 1024-thread CTAs instead (block_threads,
  // cluster = 2 so that the CTAs fill whole SM pairs). Local rows precede the GEMM in
  // its stream and take the whole device.
  const uint32_t threads = c.block_threads == 0 ? bmoe::kExThreads : c.block_threads;
  if ((threads != 256 && threads != 512 && threads != 1024) || c.cluster > 2) {
    return BMOE_INVALID_ARGUMENT;
  }
  const uint64_t sms = bmoe::device_sms();
  const uint64_t cap = c.max_ctas != 0 ? c.max_ctas
                       : (c.mode == BMOE_EP_LOCAL || c.mode == BMOE_EP_PACK)
                           ? 4 * sms
                           : (sms * 7 / 16 > 0 ? sms * 7 / 16 : 1);
  // Entries per claim: few enough that every warp of the grid gets several claims per
  // bucket (the buckets of a step hold about assignments / buckets entries each).
  const uint64_t warps_cap = cap * (threads / 32);
  const uint64_t per_bucket =
      c.assignments / ((c.mode == BMOE_EP_LOCAL || c.mode == BMOE_EP_PACK) ? 1 : c.groups) + 1;
  uint32_t span = 8;
  while (span > 1 && per_bucket / span < 4 * warps_cap) span >>= 1;
  a.span = span;
  const uint64_t want = (c.assignments + 7) / 8;   // one warp per routed row at most
  uint32_t grid = static_cast<uint32_t>(want < cap ? want : cap);
  if (grid == 0) grid = 1;  // the flags are raised even when there is nothing to send
  cudaLaunchConfig_t config{};
  config.blockDim = dim3(threads, 1, 1);
  config.dynamicSmemBytes = 0;
  config.stream = static_cast<cudaStream_t>(c.stream);
  cudaLaunchAttribute attr[1];
  if (c.cluster == 2) {
    grid = (grid + 1) / 2 * 2;
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    config.attrs = attr;
    config.numAttrs = 1;
  }
  config.gridDim = dim3(grid, 1, 1);
  a.row_bytes = c.row_bytes;
  a.status = c.status_dev;
  a.bucket_fill = c.bucket_fill_dev;
  if (c.bulk_copies != 0) {
    // one row-sized stage per warp, as many warps as fit (the bytes in flight per SM
    // bound its push rate: a row stays in its stage until NVLink has taken it)
    const uint32_t stage_bytes = (c.row_bytes + 127u) & ~127u;
    uint32_t bulk_warps = (220u * 1024u - 128u) / (stage_bytes + 12u);
    if (bulk_warps > bmoe::kBulkMaxWarps) bulk_warps = bmoe::kBulkMaxWarps;
    if (bulk_warps < 2) return BMOE_INVALID_ARGUMENT;
    const uint32_t smem = bulk_warps * stage_bytes + bulk_warps * 12 + 128;
    // per device, and cheap: set on every launch
    if (cudaFuncSetAttribute(bmoe::ep_dispatch_bulk_kernel,
                             cudaFuncAttributeMaxDynamicSharedMemorySize,
                             220 * 1024) != cudaSuccess) {
      return BMOE_CUDA_ERROR;
    }
    config.blockDim = dim3(bulk_warps * 32, 1, 1);
    config.dynamicSmemBytes = smem;
    if (cudaLaunchKernelEx(&config, bmoe::ep_dispatch_bulk_kernel, a) != cudaSuccess) {
      return BMOE_CUDA_ERROR;
    }
    return cudaPeekAtLastError() == cudaSuccess ? BMOE_OK : BMOE_CUDA_ERROR;
  }
  if (cudaLaunchKernelEx(&config, bmoe::ep_dispatch_kernel, a) != cudaSuccess) {
    return BMOE_CUDA_ERROR;
  }
  return cudaPeekAtLastError() == cudaSuccess ? BMOE_OK : BMOE_CUDA_ERROR;
}

extern "C" int bmoe_ep_return(const bmoe_ep_return_args* args) {
  if (args == nullptr) return BMOE_INVALID_ARGUMENT;
  const bmoe_ep_return_args& c = *args;
  if (c.ranks == 0 || c.self >= c.ranks || c.row_bytes == 0 || c.row_bytes % 16 != 0 ||
      c.y_bases_dev == nullptr || (c.rows != 0 && (c.d_dev == nullptr || c.origin_dev == nullptr)) ||
      (c.ranks > 1 && (c.flag_bases_dev == nullptr || c.done_counter_dev == nullptr))) {
    return BMOE_INVALID_ARGUMENT;
  }
  bmoe::ReturnArgs a;
  a.d = static_cast<const uint4*>(c.d_dev);
  a.origin = reinterpret_cast<const long long*>(c.origin_dev);
  a.y_bases = reinterpret_cast<uint4* const*>(c.y_bases_dev);
  a.flag_bases = reinterpret_cast<uint32_t* const*>(c.flag_bases_dev);
  a.done_counter = c.done_counter_dev;
  a.rows = c.rows;
  a.y_rows_cap = c.y_rows_cap;
  a.vec_per_row = c.row_bytes / 16;
  a.ranks = c.ranks;
  a.self = c.self;
  a.flag_slot = c.flag_slot;
  a.epoch = c.epoch;
  const uint64_t want = (c.rows + 7) / 8;
  const uint64_t cap = c.max_ctas != 0 ? c.max_ctas : 4ull * bmoe::device_sms();
  uint32_t grid = static_cast<uint32_t>(want < cap ? want : cap);
  if (grid == 0) grid = 1;
  bmoe::ep_return_kernel<<<grid, bmoe::kExThreads, 0, static_cast<cudaStream_t>(c.stream)>>>(a);
  return cudaPeekAtLastError() == cudaSuccess ? BMOE_OK : BMOE_CUDA_ERROR;
}

extern "C" int bmoe_ep_wait_flags(const uint32_t* flags_dev, uint32_t first_slot, uint32_t ranks,
                                  uint32_t self, uint32_t epoch, uint64_t budget_ns,
                                  uint32_t* status_dev, void* stream) {
  if (flags_dev == nullptr || ranks == 0 || ranks > 32 || self >= ranks) {
    return BMOE_INVALID_ARGUMENT;
  }
  if (ranks == 1) return BMOE_OK;  // nobody else to wait for
  if (budget_ns == 0) budget_ns = 1000000000ull;
  bmoe::ep_wait_flags_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(
      flags_dev, first_slot, ranks, self, epoch, budget_ns, status_dev);
  return cudaPeekAtLastError() == cudaSuccess ? BMOE_OK : BMOE_CUDA_ERROR;
}

extern "C" int bmoe_peer_copy_batch(const bmoe_copy_item* items, uint32_t count,
                                    void* const* streams, uint32_t stream_count) {
  if (count == 0) return BMOE_OK;
  if (items == nullptr || streams == nullptr || stream_count == 0) return BMOE_INVALID_ARGUMENT;
  for (uint32_t i = 0; i < count; ++i) {
    const bmoe_copy_item& item = items[i];
    if (item.bytes == 0) continue;
    if (item.dst == nullptr || item.src == nullptr || item.stream >= stream_count) {
      return BMOE_INVALID_ARGUMENT;
    }
    // Unified addressing tells the runtime which GPUs the two pointers live on.
    if (cudaMemcpyAsync(item.dst, item.src, item.bytes, cudaMemcpyDefault,
                        static_cast<cudaStream_t>(streams[item.stream])) != cudaSuccess) {
      return BMOE_CUDA_ERROR;
    }
  }
  return BMOE_OK;
}

namespace bmoe {
cudaError_t preload_exchange_kernels() {
  cudaError_t rc = preload_one(ep_count_kernel);
  if (rc == cudaSuccess) rc = preload_one(ep_plan_kernel);
  if (rc == cudaSuccess) rc = preload_one(ep_route_kernel);
  if (rc == cudaSuccess) rc = preload_one(ep_duplicates_kernel);
  if (rc == cudaSuccess) rc = preload_one(ep_dispatch_kernel);
  if (rc == cudaSuccess) rc = preload_one(ep_dispatch_bulk_kernel);
  if (rc == cudaSuccess) rc = preload_one(ep_return_kernel);
  if (rc == cudaSuccess) rc = preload_one(ep_wait_flags_kernel);
  return rc;
}
}  // namespace bmoe
