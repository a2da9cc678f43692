// Expert-parallel exchange overlapped with the grouped GEMM, over peer memory.
//
// Per step every rank (one GPU each)
//   1. pushes its token rows straight into the owners' expert-major packed A
//      (ep_dispatch_kernel). Experts are split into a few GROUPS in packed order;
//      the kernel works group by group and, when all of its rows of a group have
//      been written, raises a per-(group, source) flag in every peer's flag array;
//   2. runs ONE grouped GEMM whose tile scheduler holds back the tiles of a group
//      until the flags of all other sources for that group have arrived
//      (GemmParams::gate_*), so the math on early groups overlaps the transfer of
//      late ones;
//   3. pushes the result rows back to the rank each row came from
//      (ep_return_kernel, which follows the per-row origin record the dispatcher
//      left beside the row) and raises a "done" flag on every peer;
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

struct DispatchArgs {
  const uint4* x;              // [tokens, k] BF16 token rows of this rank
  const int64_t* expert_ids;   // [tokens * top_k]
  const int64_t* row_base;     // [experts] first row of (expert, this source) in the owner's A
  const int32_t* owner;        // [experts]
  const uint8_t* group_of;     // [experts] group of the expert on its owner
  uint32_t* cursor;            // [experts] rows handed out so far (zero at step start)
  uint4* const* a_bases;       // [ranks] packed A of every rank
  long long* const* origin_bases;  // [ranks] origin record per packed row
  uint32_t* const* flag_bases; // [ranks] flag arrays
  uint32_t* group_done;        // [groups] CTA arrival counters (zero at step start)
  uint32_t* chunk_next;        // [groups] next unclaimed chunk of 32 assignments (zero at start)
  int32_t* dst_rank_out;       // [assignments] or nullptr: where each assignment went
  int64_t* dst_row_out;        // [assignments] or nullptr
  uint64_t assignments;
  uint64_t rows_cap;
  uint32_t top_k;
  uint32_t vec_per_row;
  uint32_t experts;
  uint32_t ranks;
  uint32_t self;
  uint32_t groups;
  uint32_t mode;               // BMOE_EP_LOCAL / BMOE_EP_REMOTE / BMOE_EP_ALL
  uint32_t epoch;
  uint32_t span;               // assignments per claim: 32, 16, 8 or 4
};

// Group by group, a warp claims 32 consecutive assignments at a time from a shared
// counter (SMs that also push rows over NVLink or run GEMM CTAs are slower, so a
// static split would wait for them): every lane
// looks up one of them (expert, group, owner: three dependent loads, paid once per
// 32 assignments), the lanes whose assignment belongs to this pass take a row from
// the expert's cursor, and the warp then copies the selected token rows one after
// the other, 512 contiguous bytes per instruction. The row inside (expert, source)
// comes from an atomic cursor: the order of rows inside an expert does not change
// any result row, only where it sits.
__global__ void __launch_bounds__(1024) ep_dispatch_kernel(DispatchArgs a) {
  const uint32_t lane = threadIdx.x & 31;
  // Small inputs claim fewer than 32 assignments at a time so that every SM gets work.
  const uint32_t span = a.span;
  const uint32_t chunks = static_cast<uint32_t>((a.assignments + span - 1) / span);
  // Rows that stay on this rank raise no flags: one pass over all groups.
  const bool by_group = a.mode != BMOE_EP_LOCAL;
  const uint32_t passes = by_group ? a.groups : 1u;
  for (uint32_t g = 0; g < passes; ++g) {
    while (true) {
      uint32_t c = 0;
      if (lane == 0) c = atomicAdd(&a.chunk_next[g], 1u);
      c = __shfl_sync(0xffffffffu, c, 0);
      if (c >= chunks) break;
      const uint64_t i = static_cast<uint64_t>(c) * span + lane;
      int32_t to = -1;
      int64_t row = -1;
      if (lane < span && i < a.assignments) {
        const int64_t e = a.expert_ids[i];
        if (e >= 0 && e < static_cast<int64_t>(a.experts) && (!by_group || a.group_of[e] == g)) {
          const int32_t owner = a.owner[e];
          const bool local = static_cast<uint32_t>(owner) == a.self;
          const bool wanted = a.mode == BMOE_EP_ALL || (a.mode == BMOE_EP_LOCAL) == local;
          if (wanted && owner >= 0 && static_cast<uint32_t>(owner) < a.ranks) {
            row = a.row_base[e] + atomicAdd(&a.cursor[e], 1u);
            // A bad table must never become a stray access to another GPU's memory.
            if (row >= 0 && static_cast<uint64_t>(row) < a.rows_cap) {
              to = owner;
              a.origin_bases[to][row] =
                  static_cast<long long>((static_cast<uint64_t>(a.self) << kOriginRankShift) | i);
              if (a.dst_rank_out != nullptr) a.dst_rank_out[i] = to;
              if (a.dst_row_out != nullptr) a.dst_row_out[i] = row;
            }
          }
        }
      }
      uint32_t todo = __ballot_sync(0xffffffffu, to >= 0);
      while (todo != 0) {
        const uint32_t b = __ffs(todo) - 1;
        todo &= todo - 1;
        const int32_t to_b = __shfl_sync(0xffffffffu, to, b);
        const int64_t row_b = __shfl_sync(0xffffffffu, row, b);
        copy_row(a.x + ((static_cast<uint64_t>(c) * span + b) / a.top_k) * a.vec_per_row,
                 a.a_bases[to_b] + static_cast<uint64_t>(row_b) * a.vec_per_row, a.vec_per_row,
                 lane);
      }
    }
    if (by_group && a.ranks > 1) {
      signal_peers_when_grid_done(&a.group_done[g], a.flag_bases, a.ranks, a.self,
                                  g * a.ranks + a.self, a.epoch);
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

extern "C" int bmoe_ep_dispatch(const bmoe_ep_dispatch_args* args) {
  if (args == nullptr) return BMOE_INVALID_ARGUMENT;
  const bmoe_ep_dispatch_args& c = *args;
  if (c.ranks == 0 || c.self >= c.ranks || c.groups == 0 || c.groups > BMOE_EP_MAX_GROUPS ||
      c.mode > BMOE_EP_ALL || c.top_k == 0 || c.row_bytes == 0 || c.row_bytes % 16 != 0 ||
      c.a_bases_dev == nullptr || c.origin_bases_dev == nullptr || c.cursor_dev == nullptr ||
      c.row_base_dev == nullptr || c.owner_dev == nullptr || c.group_of_dev == nullptr ||
      c.chunk_next_dev == nullptr || c.assignments > 0xffffffffull * 4 ||
      (c.assignments != 0 && (c.x_dev == nullptr || c.expert_ids_dev == nullptr)) ||
      (c.ranks > 1 && c.mode != BMOE_EP_LOCAL &&
       (c.flag_bases_dev == nullptr || c.group_done_dev == nullptr))) {
    return BMOE_INVALID_ARGUMENT;
  }
  bmoe::DispatchArgs a;
  a.x = static_cast<const uint4*>(c.x_dev);
  a.expert_ids = c.expert_ids_dev;
  a.row_base = c.row_base_dev;
  a.owner = c.owner_dev;
  a.group_of = c.group_of_dev;
  a.cursor = c.cursor_dev;
  a.a_bases = reinterpret_cast<uint4* const*>(c.a_bases_dev);
  a.origin_bases = reinterpret_cast<long long* const*>(c.origin_bases_dev);
  a.flag_bases = reinterpret_cast<uint32_t* const*>(c.flag_bases_dev);
  a.group_done = c.group_done_dev;
  a.chunk_next = c.chunk_next_dev;
  a.dst_rank_out = c.dst_rank_out_dev;
  a.dst_row_out = c.dst_row_out_dev;
  a.assignments = c.assignments;
  a.rows_cap = c.rows_cap;
  a.top_k = c.top_k;
  a.vec_per_row = c.row_bytes / 16;
  a.experts = c.experts;
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
                       : c.mode == BMOE_EP_LOCAL ? 4 * sms : (sms * 7 / 16 > 0 ? sms * 7 / 16 : 1);
  // Assignments per claim: 32, or fewer when that would leave warps of the grid idle.
  const uint64_t warps_cap = cap * (threads / 32);
  uint32_t span = 32;
  while (span > 4 && (c.assignments + span - 1) / span < 2 * warps_cap) span >>= 1;
  a.span = span;
  const uint64_t per_cta = static_cast<uint64_t>(threads / 32) * span;
  const uint64_t want = (c.assignments + per_cta - 1) / per_cta;
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
