// Persistent, warp-specialised BF16 (and FP8 E4M3) grouped GEMM for sm_100a.
//
// One CTA (256 threads) per SM walks a device worklist of 20-byte tile records
// and computes, per record, a 128 x TILE_N block (one CTA) or a 256 x TILE_N
// block (a pair of CTAs in one cluster, tcgen05 cta_group::2) of
//     D_e[M_e, n] = A_e[M_e, k] * B_e[n, k]^T        (FP32 accumulate, BF16 out)
// Roles:
//   warp 0  TMA producer   A box 64x128 + B box 64xTILE_N per 64-wide k-block
//                          into a ring of SWIZZLE_128B shared-memory stages
//   warp 1  MMA issuer     tcgen05.mma 128 x TILE_N x 16, four per k-block,
//                          FP32 accumulators in Tensor Memory (two buffers)
//   warp 2  tile scheduler static stride | global atomic queue | cluster
//                          launch control; publishes decoded tile records in a
//                          small shared-memory ring read by the other roles
//   warps 4-7 epilogue     tcgen05.ld -> cvt.rn.bf16x2 -> swizzled smem ->
//                          TMA store (clipped at the expert's ragged edge)
// The k order of a tile never depends on which CTA runs it or on the scheduler,
// so all scheduling policies produce bit-identical output.
//
// Stands in for the reference's grouped kernels: the SM80 CUTLASS grouped GEMM
// (baselines/cutlass/cutlass_baseline.cu:51-80) and the TIRx variants
// (python/blackwell_moe_tirx/kernels/v1_static_ws.py:94-343 static,
// atomic_ws.py:69-271 queue, v5_clc.py:59-263 launch control).
#include "gemm_sm100.cuh"
#include "preload.cuh"

#include <cuda_runtime.h>

#include "ptx_sm100.cuh"

namespace bmoe {

namespace {

constexpr uint32_t kThreads = 256;
constexpr uint32_t kCtaRows = 128;                      // accumulator rows per CTA (TMEM lanes)
constexpr uint32_t kBlockK = 64;                        // BF16 elements per k-block (128 B)
constexpr uint32_t kABytes = kCtaRows * kBlockK * 2;    // 16 KiB
constexpr uint32_t kSchedSlots = 4;
constexpr uint32_t kEpiWarps = 4;
constexpr uint32_t kStoreCols = 64;                     // columns per TMA store box
constexpr uint32_t kStoreRows = 32;                     // rows per epilogue warp
constexpr uint32_t kStoreBytes = kStoreRows * kStoreCols * 2;  // 4 KiB
constexpr uint32_t kStagingBytes = kEpiWarps * 2 * kStoreBytes;
constexpr int32_t kSentinel = -1;

// PAIR = false: one CTA computes a 128 x TILE_N tile (tcgen05 cta_group::1).
// PAIR = true : two CTAs of a cluster compute a 256 x TILE_N tile together
//               (cta_group::2). Each CTA loads its own 128 rows of A and its
//               own half (TILE_N / 2 rows) of B and owns 128 accumulator rows;
//               the even-ranked CTA ("leader") schedules tiles and issues MMAs.
template <uint32_t TILE_N, bool PAIR>
struct Config {
  static constexpr uint32_t kGroup = PAIR ? 2 : 1;
  static constexpr uint32_t kBRows = TILE_N / kGroup;           // B rows this CTA loads
  static constexpr uint32_t kBBytes = kBRows * kBlockK * 2;
  static constexpr uint32_t kCtaStageBytes = kABytes + kBBytes;  // bytes this CTA loads
  // As many stages as 192 KiB hold: 4 of 48 KiB (128 x 256), 6 of 32 KiB (128 x 128 and
  // the pair), 8 of 24 KiB (128 x 64, the narrow tile that spreads a small-M weight
  // stream over all SMs and keeps 64 KiB of it in flight per SM).
  static constexpr uint32_t kStages = (192u * 1024u) / kCtaStageBytes;
  static constexpr uint32_t kTmemCols = 2 * TILE_N;
  // Offsets from the 1024-byte aligned base of dynamic shared memory.
  static constexpr uint32_t kOffA = 0;
  static constexpr uint32_t kOffB = kOffA + kStages * kABytes;
  static constexpr uint32_t kOffStaging = kOffB + kStages * kBBytes;
  static constexpr uint32_t kOffBarriers = kOffStaging + kStagingBytes;
  // full[S], empty[S], tmem_full[2], tmem_empty[2], sched_full[4], sched_empty[4], clc
  static constexpr uint32_t kNumBarriers = 2 * kStages + 4 + 2 * kSchedSlots + 1;
  static constexpr uint32_t kOffClcResponse = kOffBarriers + ((kNumBarriers * 8 + 15) / 16) * 16;
  static constexpr uint32_t kOffSlots = kOffClcResponse + 16;
  static constexpr uint32_t kOffMisc = kOffSlots + kSchedSlots * 32;
  static constexpr uint32_t kBytes = kOffMisc + 32;
  static constexpr uint32_t kDynamicSmem = kBytes + 1024;  // alignment slack
  // Readers of one tile-info slot: producer + 4 epilogue warps per CTA, plus
  // the MMA lane of the leader.
  static constexpr uint32_t kSlotReaders = 5 * kGroup + 1;
};

struct TileInfo {
  int32_t tile;     // worklist index or kSentinel
  uint32_t expert;
  uint32_t row0;    // first row of the tile inside the expert
  uint32_t col0;    // first output column
  uint32_t valid_m;
  uint32_t valid_n;
  uint32_t pad0;
  uint32_t pad1;
};
static_assert(sizeof(TileInfo) == 32, "slot size");

struct Misc {
  uint32_t tmem_base;
  uint32_t abort_word;
  uint32_t producer_reads;  // tile infos consumed by the producer so far
  uint32_t tiles_done;
};

__device__ __forceinline__ void report(const GemmParams& p, uint32_t site,
                                       uint32_t role, uint32_t tile, uint32_t stage,
                                       uint32_t aux) {
  if (p.status == nullptr) return;
  const uint32_t prior = atomicAdd(&p.status->count, 1u);
  if (prior == 0) {
    p.status->code = site;
    p.status->cta = blockIdx.x;
    p.status->role = role;
    p.status->tile = tile;
    p.status->stage = stage;
    p.status->aux = aux;
    __threadfence();
  }
}

// OUT_F32 = true writes the FP32 accumulators unrounded (row-major FP32 D) instead
// of BF16; everything up to the epilogue is identical.
template <uint32_t TILE_N, bool PAIR, bool OUT_F32>
__global__ void __launch_bounds__(kThreads, 1)
grouped_gemm_kernel(const __grid_constant__ GemmParams p) {
  using Cfg = Config<TILE_N, PAIR>;
  extern __shared__ uint8_t smem_raw[];
  // Swizzled TMA boxes and UMMA descriptors assume 1024-byte aligned tiles.
  const uint32_t raw_addr = ptx::smem_addr(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* const base_ptr = smem_raw + (base - raw_addr);

  const uint32_t bar0 = base + Cfg::kOffBarriers;
  auto bar_full = [&](uint32_t s) { return bar0 + 8 * s; };
  auto bar_empty = [&](uint32_t s) { return bar0 + 8 * (Cfg::kStages + s); };
  auto bar_tmem_full = [&](uint32_t b) { return bar0 + 8 * (2 * Cfg::kStages + b); };
  auto bar_tmem_empty = [&](uint32_t b) { return bar0 + 8 * (2 * Cfg::kStages + 2 + b); };
  auto bar_sched_full = [&](uint32_t s) { return bar0 + 8 * (2 * Cfg::kStages + 4 + s); };
  auto bar_sched_empty = [&](uint32_t s) {
    return bar0 + 8 * (2 * Cfg::kStages + 4 + kSchedSlots + s);
  };
  const uint32_t bar_clc = bar0 + 8 * (2 * Cfg::kStages + 4 + 2 * kSchedSlots);
  const uint32_t clc_response = base + Cfg::kOffClcResponse;
  volatile TileInfo* const slots =
      reinterpret_cast<volatile TileInfo*>(base_ptr + Cfg::kOffSlots);
  volatile Misc* const misc = reinterpret_cast<volatile Misc*>(base_ptr + Cfg::kOffMisc);
  volatile uint32_t* const abort_word = &misc->abort_word;

  const uint32_t warp = threadIdx.x >> 5;
  const uint32_t lane = threadIdx.x & 31;
  const uint64_t budget = p.wait_budget_ns;

  // Position inside the pair and the scheduling unit (CTA or CTA pair).
  const uint32_t cta_rank = PAIR ? ptx::cluster_cta_rank() : 0u;
  const bool leader = cta_rank == 0;
  const uint32_t unit = PAIR ? blockIdx.x / 2 : blockIdx.x;
  const uint32_t units = PAIR ? gridDim.x / 2 : gridDim.x;
  // Tile total: a launch parameter, or read from where the worklist builder left it.
  uint32_t tile_count = p.tile_count;
  uint32_t main_end = p.main_end;
  if (p.tile_count_dev != nullptr) {
    const uint32_t on_device = *p.tile_count_dev;
    tile_count = on_device < p.tile_count ? on_device : p.tile_count;
    main_end = tile_count;
  }

  // Barrier helpers that hide where the barrier lives. In pair mode the
  // operand-full, accumulator-empty and slot-empty barriers of the LEADER are
  // the live ones; the peer reaches them through cluster addresses.
  auto wait = [&](uint32_t bar, uint32_t parity) -> bool {
    if constexpr (PAIR) {
      return ptx::mbar_wait_cluster(bar, parity, abort_word, budget);
    } else {
      return ptx::mbar_wait(bar, parity, abort_word, budget);
    }
  };
  auto arrive_at_leader = [&](uint32_t bar) {
    if constexpr (PAIR) {
      ptx::mbar_arrive_cluster(ptx::map_to_cta(bar, 0));
    } else {
      ptx::mbar_arrive(bar);
    }
  };

  // Optional per-CTA wait accounting (cycles spent blocked, per role and
  // barrier kind); costs one predictable branch per wait when disabled.
  const bool tracing = p.trace != nullptr;
  auto timed_wait = [&](uint32_t bar, uint32_t parity, uint64_t& bucket) -> bool {
    if (!tracing) return wait(bar, parity);
    const long long t0 = clock64();
    const bool ok = wait(bar, parity);
    bucket += static_cast<uint64_t>(clock64() - t0);
    return ok;
  };
  const long long kernel_t0 = tracing ? clock64() : 0;

  // The first tile of a unit is known before any set-up (static stride and launch
  // control start at the unit's own index, the queue's first claim needs nothing but the
  // counter): the scheduler lane fetches it, and warms the descriptors it needs, while
  // barriers and Tensor Memory are being set up. A small problem is one tile per CTA, so
  // this takes the two dependent global reads off the front of the launch.
  bmoe_tile first_rec{};
  uint32_t first_index = 0xffffffffu;   // worklist index of first_rec, if fetched
  uint32_t first_claim = 0;             // queue mode: the claim made ahead of the set-up
  if (warp == 2 && lane == 0 && leader) {
    if (p.sched_mode == kSchedQueue) {
      first_claim = atomicAdd(&p.queue[0], p.claim_size);
      if (first_claim < main_end) first_index = first_claim;
    } else if (unit < tile_count) {
      first_index = unit;
    }
    if (first_index != 0xffffffffu) {
      first_rec = p.tiles[first_index];
      const uint32_t e = first_rec.expert_id;
      ptx::tensormap_prefetch(p.a_row_offsets != nullptr ? p.tmap_a : p.tmap_a + e);
      ptx::tensormap_prefetch(p.tmap_b + e);
      if (p.push_origin == nullptr) ptx::tensormap_prefetch(p.tmap_d + e);
    }
  }

  // ------------------------------------------------------------- set-up --
  if (threadIdx.x == 0) {
    for (uint32_t s = 0; s < Cfg::kStages; ++s) {
      ptx::mbar_init(bar_full(s), 1);
      ptx::mbar_init(bar_empty(s), 1);
    }
    for (uint32_t b = 0; b < 2; ++b) {
      ptx::mbar_init(bar_tmem_full(b), 1);
      ptx::mbar_init(bar_tmem_empty(b), kEpiWarps * Cfg::kGroup);
    }
    for (uint32_t s = 0; s < kSchedSlots; ++s) {
      ptx::mbar_init(bar_sched_full(s), 1);
      ptx::mbar_init(bar_sched_empty(s), Cfg::kSlotReaders);
    }
    ptx::mbar_init(bar_clc, 1);
    misc->abort_word = 0;
    misc->producer_reads = 0;
    misc->tiles_done = 0;
    ptx::fence_barrier_init();
  }
  if (warp == 1) {
    if constexpr (PAIR) {
      ptx::tmem_alloc_pair(base + Cfg::kOffMisc, Cfg::kTmemCols);  // -> misc->tmem_base
      ptx::tmem_relinquish_pair();
    } else {
      ptx::tmem_alloc(base + Cfg::kOffMisc, Cfg::kTmemCols);
      ptx::tmem_relinquish();
    }
  }
  ptx::tc_fence_before_sync();
  if constexpr (PAIR) {
    ptx::cluster_sync();  // both CTAs' barriers exist before any remote arrive
  } else {
    __syncthreads();
  }
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = misc->tmem_base;
  // time line of the CTA for the trace (cycles since the kernel's first instruction)
  const uint64_t stamp_setup = tracing ? static_cast<uint64_t>(clock64() - kernel_t0) : 0;

  // ---------------------------------------------------------- scheduler --
  if (warp == 2) {
    if (lane == 0 && leader) {
      uint32_t published = 0;
      bool alive = true;
      const uint32_t peer_slots = PAIR ? ptx::map_to_cta(base + Cfg::kOffSlots, 1) : 0u;
      // Publishes one decoded record (or the sentinel) to the next ring slot
      // (of both CTAs in pair mode).
      // Groups whose rows are known to have arrived from every other rank.
      uint32_t groups_ready = 0;
      auto gate = [&](uint32_t expert) -> bool {
        const uint32_t g = p.gate_group_of[expert];
        if (g >= 32 || ((groups_ready >> g) & 1u) != 0) return true;
        uint64_t start = 0;
        // plane 0: rows pushed by the sources' SMs; plane 1: rows sent as peer copies
        const uint32_t copy_mask = p.gate_copy_mask != nullptr ? p.gate_copy_mask[g] : 0u;
        for (uint32_t plane = 0; plane < 2; ++plane) {
          if (plane == 1 && copy_mask == 0) break;
          for (uint32_t r = 0; r < p.gate_ranks; ++r) {
            if (r == p.gate_self) continue;
            if (plane == 1 && ((copy_mask >> r) & 1u) == 0) continue;
            const uint32_t* flag =
                p.gate_flags + plane * p.gate_copy_plane + g * p.gate_ranks + r;
            for (uint32_t spin = 1;; ++spin) {
              if (static_cast<int32_t>(ptx::ld_acquire_sys_u32(flag) - p.gate_epoch) >= 0) break;
              if ((spin & 0xf) == 0) {
                if (*abort_word != 0) return false;
                const uint64_t now = ptx::global_timer_ns();
                if (start == 0) {
                  start = now;
                } else if (now - start > budget) {
                  *abort_word = 1;
                  report(p, kSiteSchedGate, 0, expert, g, r | (plane << 8));
                  return false;
                }
              }
              __nanosleep(200);
            }
          }
        }
        if (p.expand_records != nullptr && g < p.expand_groups) {
          // rows of this group that the sources did not send: copied here, by warp 3 of
          // the CTAs of this launch, from the rows that did arrive
          uint32_t want = 0;
          for (uint32_t r = 0; r < p.gate_ranks; ++r) {
            if (r != p.gate_self) want += p.expand_count[g * p.gate_ranks + r];
          }
          for (uint32_t spin = 1;; ++spin) {
            if (ptx::ld_acquire_gpu_u32(p.expand_done + g) >= want) break;
            if ((spin & 0xf) == 0) {
              if (*abort_word != 0) return false;
              const uint64_t now = ptx::global_timer_ns();
              if (start == 0) {
                start = now;
              } else if (now - start > budget) {
                *abort_word = 1;
                report(p, kSiteSchedExpand, 0, expert, g, want);
                return false;
              }
            }
            __nanosleep(100);
          }
        }
        // The rows were written by other GPUs' ordinary stores; the TMA loads that
        // follow (async proxy) must observe them.
        ptx::fence_proxy_async_all();
        groups_ready |= 1u << g;
        return true;
      };
      auto publish = [&](int32_t tile_index) -> bool {
        const uint32_t slot = published % kSchedSlots;
        const uint32_t round = (published / kSchedSlots) & 1u;
        bmoe_tile t{};
        if (tile_index != kSentinel) {
#ifdef BMOE_CHECKS
          if (static_cast<uint32_t>(tile_index) < tile_count)   // else: reported below, not read
#endif
          t = static_cast<uint32_t>(tile_index) == first_index ? first_rec : p.tiles[tile_index];
        }
#ifdef BMOE_CHECKS
        if (tile_index != kSentinel) {
          uint32_t failed = 0, value = 0;
          const uint32_t tile_rows = kCtaRows * Cfg::kGroup;
          if (static_cast<uint32_t>(tile_index) >= tile_count) {
            failed = kCheckTileIndex; value = static_cast<uint32_t>(tile_index);
          } else if (t.expert_id >= p.check_experts) {
            failed = kCheckExpert; value = t.expert_id;
          } else if (t.valid_n == 0 || t.valid_n > TILE_N ||
                     static_cast<uint64_t>(t.tile_n) * TILE_N + t.valid_n > p.check_n) {
            failed = kCheckColumns; value = t.tile_n;
          } else if (t.valid_m == 0 || t.valid_m > tile_rows) {
            failed = kCheckRows; value = t.valid_m;
          } else if (p.a_row_offsets != nullptr &&
                     p.a_row_offsets[t.expert_id] + static_cast<uint64_t>(t.tile_m) * tile_rows +
                             t.valid_m > p.check_a_rows) {
            failed = kCheckPackedRows; value = t.tile_m;
          } else if (static_cast<uint64_t>(p.k_blocks) * 128u < p.check_k_bytes ||
                     static_cast<uint64_t>(p.k_blocks - 1) * 128u >= p.check_k_bytes) {
            failed = kCheckKBlocks; value = p.k_blocks;
          } else if (2 * TILE_N > Cfg::kTmemCols) {
            failed = kCheckTmemColumns; value = 2 * TILE_N;
          }
          if (failed != 0) {
            *abort_word = 1;
            report(p, kSiteCheck, 0, static_cast<uint32_t>(tile_index), failed, value);
            return false;
          }
        }
#endif
        if (p.gate_flags != nullptr && tile_index != kSentinel && !gate(t.expert_id)) {
          return false;
        }
        if (!wait(bar_sched_empty(slot), round ^ 1u)) {
          report(p, kSiteSchedSlot, 0, static_cast<uint32_t>(tile_index), slot, published);
          return false;
        }
        TileInfo rec{};
        rec.tile = tile_index;
        if (tile_index != kSentinel) {
          rec.expert = t.expert_id;
          rec.row0 = t.tile_m * (kCtaRows * Cfg::kGroup);
          rec.col0 = t.tile_n * TILE_N;
          rec.valid_m = t.valid_m;
          rec.valid_n = t.valid_n;
        }
        volatile TileInfo* info = &slots[slot];
        info->tile = rec.tile;
        info->expert = rec.expert;
        info->row0 = rec.row0;
        info->col0 = rec.col0;
        info->valid_m = rec.valid_m;
        info->valid_n = rec.valid_n;
        ptx::mbar_arrive(bar_sched_full(slot));
        if constexpr (PAIR) {
          const uint32_t remote = peer_slots + slot * 32;
          ptx::st_cluster_u32(remote + 0, static_cast<uint32_t>(rec.tile));
          ptx::st_cluster_u32(remote + 4, rec.expert);
          ptx::st_cluster_u32(remote + 8, rec.row0);
          ptx::st_cluster_u32(remote + 12, rec.col0);
          ptx::st_cluster_u32(remote + 16, rec.valid_m);
          ptx::st_cluster_u32(remote + 20, rec.valid_n);
          ptx::mbar_arrive_cluster(ptx::map_to_cta(bar_sched_full(slot), 1));  // release
        }
        ++published;
        return true;
      };
      // Claims are throttled so that at most `lookahead` published tiles are
      // still unread by the producer; this keeps late tiles stealable.
      auto pace = [&]() -> bool {
        if (p.lookahead == 0) return true;
        uint64_t start = 0;
        for (uint32_t spin = 1;; ++spin) {
          if (published - misc->producer_reads < p.lookahead) return true;
          if ((spin & 0x3f) == 0) {
            if (*abort_word != 0) return false;
            const uint64_t now = ptx::global_timer_ns();
            if (start == 0) {
              start = now;
            } else if (now - start > budget) {
              *abort_word = 1;
              report(p, kSiteSchedPace, 0, published, 0, misc->producer_reads);
              return false;
            }
          }
          __nanosleep(64);
        }
      };

      if (p.sched_mode == kSchedStatic) {
        for (uint32_t t = unit; alive && t < tile_count; t += units) {
          alive = publish(static_cast<int32_t>(t));
        }
      } else if (p.sched_mode == kSchedQueue) {
        // Main part: chunks of claim_size below main_end (the first claim was made
        // before the set-up).
        bool claimed_ahead = true;
        while (alive) {
          if (!pace()) { alive = false; break; }
          const uint32_t begin = claimed_ahead ? first_claim : atomicAdd(&p.queue[0], p.claim_size);
          claimed_ahead = false;
          if (begin >= main_end) break;
          const uint32_t end = min(begin + p.claim_size, main_end);
          for (uint32_t t = begin; alive && t < end; ++t) {
            if (t != begin && !pace()) { alive = false; break; }
            alive = publish(static_cast<int32_t>(t));
          }
        }
        // Tail part: single tiles from the second counter.
        while (alive) {
          if (!pace()) { alive = false; break; }
          const uint32_t t = atomicAdd(&p.queue[1], 1u);
          if (t >= tile_count) break;
          alive = publish(static_cast<int32_t>(t));
        }
      } else {  // kSchedClc: one CTA (pair) per tile, steal units not yet started
        uint32_t clc_round = 0;
        uint32_t t = unit;
        if (t < tile_count) alive = publish(static_cast<int32_t>(t));
        while (alive) {
          if (!pace()) { alive = false; break; }
          ptx::mbar_arrive_expect_tx(bar_clc, 16);
          ptx::clc_try_cancel(clc_response, bar_clc);
          if (!ptx::mbar_wait(bar_clc, clc_round, abort_word, budget)) {
            report(p, kSiteSchedClc, 0, t, 0, published);
            alive = false;
            break;
          }
          clc_round ^= 1u;
          uint32_t stolen = 0;
          const bool got = ptx::clc_query(clc_response, &stolen);
          ptx::fence_async_shared();
          if (!got) break;  // no pending unit left; must not ask again
          t = PAIR ? stolen / 2 : stolen;
          if (t < tile_count) alive = publish(static_cast<int32_t>(t));
        }
      }
      if (alive) publish(kSentinel);
    }
    __syncwarp();
  }

  // ----------------------------------------------------------- producer --
  // The whole warp walks the loop converged; one elected lane issues the
  // arrivals and the TMA loads.
  else if (warp == 0) {
    uint32_t reads = 0;
    uint32_t stage = 0, stage_round = 0;
    uint32_t last_expert = 0xffffffffu;
    uint64_t t_info = 0, t_stage = 0;
    // bytes that land per stage: the A box (possibly fewer than 128 rows) and the B box
    const uint32_t tx_bytes = (p.a_box_bytes + Cfg::kBBytes) * Cfg::kGroup;
    const uint32_t k_block_elems = p.fp8 != 0 ? 2 * kBlockK : kBlockK;   // 128 bytes of a row
    while (true) {
      const uint32_t slot = reads % kSchedSlots;
      const uint32_t round = (reads / kSchedSlots) & 1u;
      if (!timed_wait(bar_sched_full(slot), round, t_info)) {
        if (lane == 0) report(p, kSiteProducerInfo, 1, reads, slot, 0);
        break;
      }
      const int32_t tile = slots[slot].tile;
      const uint32_t expert = slots[slot].expert;
      const uint32_t row0 = slots[slot].row0 + cta_rank * kCtaRows;
      const uint32_t col0 = slots[slot].col0 + cta_rank * Cfg::kBRows;
      __syncwarp();
      ++reads;
      if (ptx::elect_one()) {
        arrive_at_leader(bar_sched_empty(slot));
        if (leader) misc->producer_reads = reads;
      }
      if (tile == kSentinel) break;

      const bool packed_a = p.a_row_offsets != nullptr;
      const CUtensorMap* const map_a = packed_a ? p.tmap_a : p.tmap_a + expert;
      const CUtensorMap* const map_b = p.tmap_b + expert;
      const uint32_t a_row0 =
          packed_a ? row0 + static_cast<uint32_t>(p.a_row_offsets[expert]) : row0;
      // Gated launch: the rows of this tile were stored by other GPUs; order this
      // warp's TMA loads after the scheduler's observation of their flags.
      if (p.gate_flags != nullptr) ptx::fence_proxy_async_all();
      if (expert != last_expert) {
        if (ptx::elect_one()) {
          ptx::tensormap_acquire(map_a);
          ptx::tensormap_acquire(map_b);
        }
        last_expert = expert;
      }
      bool ok = true;
      for (uint32_t kb = 0; kb < p.k_blocks; ++kb) {
        if (!timed_wait(bar_empty(stage), stage_round ^ 1u, t_stage)) {
          if (lane == 0) {
            report(p, kSiteProducerStage, 1, static_cast<uint32_t>(tile), stage, kb);
          }
          ok = false;
          break;
        }
        const uint32_t dst_a = base + Cfg::kOffA + stage * kABytes;
        const uint32_t dst_b = base + Cfg::kOffB + stage * Cfg::kBBytes;
        const int32_t k0 = static_cast<int32_t>(kb * k_block_elems);   // element coordinate
        if (ptx::elect_one()) {
          if constexpr (PAIR) {
            // Both CTAs' bytes are counted on the leader's barrier.
            if (leader) ptx::mbar_arrive_expect_tx(bar_full(stage), tx_bytes);
            const uint32_t full = ptx::map_to_cta(bar_full(stage), 0);
            ptx::tma_load_2d_pair(dst_a, map_a, full, k0, static_cast<int32_t>(a_row0));
            ptx::tma_load_2d_pair(dst_b, map_b, full, k0, static_cast<int32_t>(col0));
          } else {
            ptx::mbar_arrive_expect_tx(bar_full(stage), tx_bytes);
            ptx::tma_load_2d(dst_a, map_a, bar_full(stage), k0, static_cast<int32_t>(a_row0));
            ptx::tma_load_2d(dst_b, map_b, bar_full(stage), k0, static_cast<int32_t>(col0));
          }
        }
        if (++stage == Cfg::kStages) { stage = 0; stage_round ^= 1u; }
      }
      if (!ok) break;
    }
    if (tracing && lane == 0) {
      p.trace[blockIdx.x * kTraceWords + 0] = t_info;
      p.trace[blockIdx.x * kTraceWords + 1] = t_stage;
    }
    __syncwarp();
  }

  // ---------------------------------------------------------------- MMA --
  // Leader CTA only. The warp stays converged; one elected lane (always the
  // same one, so tcgen05.commit covers its MMAs) issues the tensor-core work.
  else if (warp == 1) {
    if (leader) {
      constexpr uint32_t idesc = ptx::make_bf16_idesc(kCtaRows * Cfg::kGroup, TILE_N);
      constexpr uint32_t idesc_fp8 = ptx::make_e4m3_idesc(kCtaRows * Cfg::kGroup, TILE_N);
      const bool fp8 = p.fp8 != 0;
      uint32_t reads = 0;
      uint32_t stage = 0, stage_round = 0;
      uint32_t buf = 0, buf_round = 0;
      uint64_t t_info = 0, t_accum = 0, t_operands = 0, t_issue = 0;
      uint64_t stamp_first_operands = 0, stamp_last_issue = 0;
      while (true) {
        const uint32_t slot = reads % kSchedSlots;
        const uint32_t round = (reads / kSchedSlots) & 1u;
        if (!timed_wait(bar_sched_full(slot), round, t_info)) {
          if (lane == 0) report(p, kSiteMmaInfo, 2, reads, slot, 0);
          break;
        }
        const int32_t tile = slots[slot].tile;
        __syncwarp();
        if (ptx::elect_one()) ptx::mbar_arrive(bar_sched_empty(slot));
        ++reads;
        if (tile == kSentinel) break;

        // The epilogue(s) must have drained this accumulator buffer.
        if (!timed_wait(bar_tmem_empty(buf), buf_round ^ 1u, t_accum)) {
          if (lane == 0) report(p, kSiteMmaAccum, 2, static_cast<uint32_t>(tile), buf, 0);
          break;
        }
        ptx::tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + buf * TILE_N;
        bool ok = true;
        for (uint32_t kb = 0; kb < p.k_blocks; ++kb) {
          if (!timed_wait(bar_full(stage), stage_round, t_operands)) {
            if (lane == 0) {
              report(p, kSiteMmaStage, 2, static_cast<uint32_t>(tile), stage, kb);
            }
            ok = false;
            break;
          }
          ptx::tc_fence_after_sync();
          if (tracing && stamp_first_operands == 0) {
            stamp_first_operands = static_cast<uint64_t>(clock64() - kernel_t0);
          }
          const uint64_t a_desc =
              ptx::make_kmajor_sw128_desc(base + Cfg::kOffA + stage * kABytes);
          const uint64_t b_desc =
              ptx::make_kmajor_sw128_desc(base + Cfg::kOffB + stage * Cfg::kBBytes);
          const long long issue_t0 = tracing ? clock64() : 0;
          if (ptx::elect_one()) {
            if (!fp8) {
#pragma unroll
              for (uint32_t ks = 0; ks < kBlockK / 16; ++ks) {
                // 16 BF16 = 32 bytes along k inside the 128-byte swizzle row.
                const uint32_t acc = (kb | ks) != 0 ? 1u : 0u;
                if constexpr (PAIR) {
                  ptx::umma_bf16_ss_pair(d_tmem, a_desc + 2 * ks, b_desc + 2 * ks, idesc, acc);
                } else {
                  ptx::umma_bf16_ss(d_tmem, a_desc + 2 * ks, b_desc + 2 * ks, idesc, acc);
                }
              }
            } else {
#pragma unroll
              for (uint32_t ks = 0; ks < kBlockK / 16; ++ks) {
                // 32 FP8 = the same 32 bytes.
                const uint32_t acc = (kb | ks) != 0 ? 1u : 0u;
                if constexpr (PAIR) {
                  ptx::umma_e4m3_ss_pair(d_tmem, a_desc + 2 * ks, b_desc + 2 * ks, idesc_fp8,
                                         acc);
                } else {
                  ptx::umma_e4m3_ss(d_tmem, a_desc + 2 * ks, b_desc + 2 * ks, idesc_fp8, acc);
                }
              }
            }
            // The stage is reusable (in both CTAs) once these MMAs retire.
            if constexpr (PAIR) {
              ptx::umma_commit_pair(bar_empty(stage));
              ptx::umma_commit_pair(ptx::map_to_cta(bar_empty(stage), 1));
            } else {
              ptx::umma_commit(bar_empty(stage));
            }
            if (kb + 1 == p.k_blocks) {
              // Accumulator complete: wake the epilogue of both CTAs.
              if constexpr (PAIR) {
                ptx::umma_commit_pair(bar_tmem_full(buf));
                ptx::umma_commit_pair(ptx::map_to_cta(bar_tmem_full(buf), 1));
              } else {
                ptx::umma_commit(bar_tmem_full(buf));
              }
            }
          }
          if (tracing) {
            const long long now = clock64();
            t_issue += static_cast<uint64_t>(now - issue_t0);
            stamp_last_issue = static_cast<uint64_t>(now - kernel_t0);
          }
          if (++stage == Cfg::kStages) { stage = 0; stage_round ^= 1u; }
        }
        if (!ok) break;
        if (++buf == 2) { buf = 0; buf_round ^= 1u; }
      }
      if (tracing && lane == 0) {
        p.trace[blockIdx.x * kTraceWords + 2] = t_info;
        p.trace[blockIdx.x * kTraceWords + 3] = t_accum;
        p.trace[blockIdx.x * kTraceWords + 4] = t_operands;
        p.trace[blockIdx.x * kTraceWords + 10] = t_issue;
        p.trace[blockIdx.x * kTraceWords + 11] = stamp_setup;
        p.trace[blockIdx.x * kTraceWords + 12] = stamp_first_operands;
        p.trace[blockIdx.x * kTraceWords + 13] = stamp_last_issue;
      }
    }
    __syncwarp();
  }

  // ------------------------------------------------------- row expansion --
  // Send-once exchange: group by group and source by source, wait for the source's flag,
  // then copy primary rows onto the rows of the duplicates, a few records per claim, in
  // competition with warp 3 of every other CTA of the launch.
  else if (warp == 3) {
    if (p.expand_records != nullptr && p.gate_flags != nullptr) {
      constexpr uint32_t kClaim = 2;
      bool alive = true;
      for (uint32_t g = 0; alive && g < p.expand_groups; ++g) {
        for (uint32_t r = 0; alive && r < p.gate_ranks; ++r) {
          if (r == p.gate_self) continue;
          const uint32_t list = g * p.gate_ranks + r;
          uint32_t ok = 1;
          if (lane == 0) {
            const uint32_t* flag = p.gate_flags + list;
            uint64_t start = 0;
            for (uint32_t spin = 1;; ++spin) {
              if (static_cast<int32_t>(ptx::ld_acquire_sys_u32(flag) - p.gate_epoch) >= 0) break;
              if ((spin & 0xf) == 0) {
                if (*abort_word != 0) { ok = 0; break; }
                const uint64_t now = ptx::global_timer_ns();
                if (start == 0) {
                  start = now;
                } else if (now - start > budget) {
                  *abort_word = 1;
                  report(p, kSiteExpandFlag, 4, 0, g, r);
                  ok = 0;
                  break;
                }
              }
              __nanosleep(500);
            }
          }
          ok = __shfl_sync(0xffffffffu, ok, 0);
          if (ok == 0) { alive = false; break; }
          uint32_t count = lane == 0 ? p.expand_count[list] : 0u;
          count = __shfl_sync(0xffffffffu, count, 0);
          if (count > p.expand_cap) count = p.expand_cap;
          const uint2* const records = p.expand_records + static_cast<size_t>(list) * p.expand_cap;
          while (true) {
            uint32_t at = 0;
            if (lane == 0) at = atomicAdd(&p.expand_next[list], kClaim);
            at = __shfl_sync(0xffffffffu, at, 0);
            if (at >= count) break;
            const uint32_t end = min(at + kClaim, count);
            for (uint32_t i = at; i < end; ++i) {
              const uint2 rec = records[i];
              if (rec.x < p.expand_rows_cap && rec.y < p.expand_rows_cap) {
                const uint4* src = p.expand_a + static_cast<size_t>(rec.x) * p.expand_vec_per_row;
                uint4* dst = p.expand_a + static_cast<size_t>(rec.y) * p.expand_vec_per_row;
                for (uint32_t v0 = 0; v0 < p.expand_vec_per_row; v0 += 32 * 8) {
                  uint4 regs[8];
#pragma unroll
                  for (uint32_t u = 0; u < 8; ++u) {
                    const uint32_t v = v0 + u * 32 + lane;
                    if (v < p.expand_vec_per_row) regs[u] = src[v];
                  }
#pragma unroll
                  for (uint32_t u = 0; u < 8; ++u) {
                    const uint32_t v = v0 + u * 32 + lane;
                    if (v < p.expand_vec_per_row) dst[v] = regs[u];
                  }
                }
              }
            }
            // the copies are visible device-wide before they are counted
            __threadfence();
            __syncwarp();
            if (lane == 0) atomicAdd(&p.expand_done[g], end - at);
          }
        }
      }
    }
    __syncwarp();
  }

  // ----------------------------------------------------------- epilogue --
  else if (warp >= 4) {
    const uint32_t quad = warp & 3u;  // TMEM lane quadrant this warp may read
    const uint32_t staging = base + Cfg::kOffStaging + quad * 2 * kStoreBytes;
    const uint32_t row_in_tile = cta_rank * kCtaRows + quad * kStoreRows;
    uint64_t stamp_last_accum = 0;
    uint32_t reads = 0;
    uint32_t buf = 0, buf_round = 0;
    uint32_t sbuf = 0;
    uint32_t last_expert = 0xffffffffu;
    uint32_t tiles_done = 0;
    uint64_t t_info = 0, t_accum = 0, t_drain = 0;
    while (true) {
      const uint32_t slot = reads % kSchedSlots;
      const uint32_t round = (reads / kSchedSlots) & 1u;
      if (!timed_wait(bar_sched_full(slot), round, t_info)) {
        if (lane == 0 && quad == 0) report(p, kSiteEpiInfo, 3, reads, slot, 0);
        break;
      }
      const int32_t tile = slots[slot].tile;
      const uint32_t expert = slots[slot].expert;
      const uint32_t row0 = slots[slot].row0;
      const uint32_t col0 = slots[slot].col0;
      const uint32_t valid_m = slots[slot].valid_m;
      const uint32_t valid_n = slots[slot].valid_n;
      __syncwarp();
      if (lane == 0) arrive_at_leader(bar_sched_empty(slot));
      ++reads;
      if (tile == kSentinel) break;

      // Push mode: where this lane's row goes (looked up while the MMAs still run).
      uint4* push_dst = nullptr;
      if constexpr (!OUT_F32) {
        if (p.push_origin != nullptr && row_in_tile + lane < valid_m) {
          const uint64_t rec = static_cast<uint64_t>(
              p.push_origin[p.push_expert_row[expert] + row0 + row_in_tile + lane]);
          const uint64_t to = rec >> 40;
          const uint64_t at = rec & ((1ull << 40) - 1);
          // A bad record must never become a stray access to another GPU's memory.
          if (to < p.push_ranks && at < p.push_rows_cap) {
            push_dst = p.push_bases[to] + at * p.push_vec_per_row + (col0 >> 3);
          }
        }
      }

      if (!timed_wait(bar_tmem_full(buf), buf_round, t_accum)) {
        if (lane == 0 && quad == 0) {
          report(p, kSiteEpiAccum, 3, static_cast<uint32_t>(tile), buf, 0);
        }
        break;
      }
      ptx::tc_fence_after_sync();
      if (tracing) stamp_last_accum = static_cast<uint64_t>(clock64() - kernel_t0);

      const CUtensorMap* const map_d = p.tmap_d + expert;
      if (lane == 0 && expert != last_expert) ptx::tensormap_acquire(map_d);
      last_expert = expert;

      const bool has_rows = row_in_tile < valid_m;
      // One store box is 128 bytes wide: 64 BF16 or 32 FP32 columns.
      constexpr uint32_t kChunkCols = OUT_F32 ? 32u : kStoreCols;
      const uint32_t chunks = has_rows ? (valid_n + kChunkCols - 1) / kChunkCols : 0;
      const uint32_t lane_taddr = tmem_base + ((quad * 32u) << 16) + buf * TILE_N;
      const long long drain_t0 = tracing ? clock64() : 0;
      for (uint32_t c = 0; c < chunks; ++c) {
        uint32_t lo[32], hi[32];
        ptx::tmem_load_32x32(lane_taddr + c * kChunkCols, lo);
        if constexpr (!OUT_F32) ptx::tmem_load_32x32(lane_taddr + c * kChunkCols + 32, hi);
        ptx::tmem_load_wait();
        if (c + 1 == chunks) {
          // All of this warp's accumulator rows are in registers: hand the
          // buffer back before the (slower) conversion and store.
          ptx::tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) arrive_at_leader(bar_tmem_empty(buf));
        }
        // The store issued two chunks ago read from this staging buffer.
        if (lane == 0) ptx::tma_store_wait_read<1>();
        __syncwarp();
        const uint32_t row_smem = staging + sbuf * kStoreBytes + lane * 128u;
        const uint32_t sw = lane & 7u;
        if constexpr (OUT_F32) {
#pragma unroll
          for (uint32_t j = 0; j < 8; ++j) {
            ptx::st_shared_v4(row_smem + ((j ^ sw) << 4), lo[4 * j + 0], lo[4 * j + 1],
                              lo[4 * j + 2], lo[4 * j + 3]);
          }
        } else {
#pragma unroll
          for (uint32_t j = 0; j < 4; ++j) {
            ptx::st_shared_v4(
                row_smem + ((j ^ sw) << 4),
                ptx::pack_bf16x2(__uint_as_float(lo[8 * j + 0]), __uint_as_float(lo[8 * j + 1])),
                ptx::pack_bf16x2(__uint_as_float(lo[8 * j + 2]), __uint_as_float(lo[8 * j + 3])),
                ptx::pack_bf16x2(__uint_as_float(lo[8 * j + 4]), __uint_as_float(lo[8 * j + 5])),
                ptx::pack_bf16x2(__uint_as_float(lo[8 * j + 6]), __uint_as_float(lo[8 * j + 7])));
          }
#pragma unroll
          for (uint32_t j = 0; j < 4; ++j) {
            ptx::st_shared_v4(
                row_smem + (((j + 4) ^ sw) << 4),
                ptx::pack_bf16x2(__uint_as_float(hi[8 * j + 0]), __uint_as_float(hi[8 * j + 1])),
                ptx::pack_bf16x2(__uint_as_float(hi[8 * j + 2]), __uint_as_float(hi[8 * j + 3])),
                ptx::pack_bf16x2(__uint_as_float(hi[8 * j + 4]), __uint_as_float(hi[8 * j + 5])),
                ptx::pack_bf16x2(__uint_as_float(hi[8 * j + 6]), __uint_as_float(hi[8 * j + 7])));
          }
        }
        if constexpr (!OUT_F32) {
          if (p.push_origin != nullptr) {
            // Rows leave from the staging tile: 8 lanes write the 128 bytes of one row.
            __syncwarp();
            const uint32_t tile_smem = staging + sbuf * kStoreBytes;
#pragma unroll
            for (uint32_t it = 0; it < 8; ++it) {
              const uint32_t r = it * 4 + (lane >> 3);
              const uint32_t j = lane & 7u;
              const unsigned long long dst_r = __shfl_sync(
                  0xffffffffu, reinterpret_cast<unsigned long long>(push_dst), r);
              if (dst_r != 0 && c * kChunkCols + j * 8 < valid_n) {
                const uint4 v = ptx::ld_shared_v4(tile_smem + r * 128u + ((j ^ (r & 7u)) << 4));
                reinterpret_cast<uint4*>(dst_r)[c * (kChunkCols / 8) + j] = v;
              }
            }
            sbuf ^= 1u;
            continue;
          }
        }
        ptx::fence_async_shared();
        __syncwarp();
        if (lane == 0) {
          ptx::tma_store_2d(map_d, staging + sbuf * kStoreBytes,
                            static_cast<int32_t>(col0 + c * kChunkCols),
                            static_cast<int32_t>(row0 + row_in_tile));
          ptx::tma_store_commit();
        }
        sbuf ^= 1u;
      }
      if (chunks == 0) {
        // Nothing to read for this warp (rows beyond the ragged edge).
        ptx::tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) arrive_at_leader(bar_tmem_empty(buf));
      }
      if (tracing) t_drain += static_cast<uint64_t>(clock64() - drain_t0);
      if (++buf == 2) { buf = 0; buf_round ^= 1u; }
      ++tiles_done;
      if (leader && quad == 0 && lane == 0 && p.tile_visits != nullptr) {
        atomicAdd(&p.tile_visits[tile], 1u);
      }
    }
    if (lane == 0) ptx::tma_store_wait_all();
    // Pushed rows may sit in other GPUs' memory: make them visible system-wide
    // before the kernel ends and the next launch in the stream raises the flags.
    if (p.push_origin != nullptr) __threadfence_system();
    if (quad == 0 && lane == 0) misc->tiles_done = tiles_done;
    if (tracing && quad == 0 && lane == 0) {
      p.trace[blockIdx.x * kTraceWords + 5] = t_info;
      p.trace[blockIdx.x * kTraceWords + 6] = t_accum;
      p.trace[blockIdx.x * kTraceWords + 7] = t_drain;
      p.trace[blockIdx.x * kTraceWords + 8] = tiles_done;
      p.trace[blockIdx.x * kTraceWords + 14] = stamp_last_accum;
      p.trace[blockIdx.x * kTraceWords + 15] = static_cast<uint64_t>(clock64() - kernel_t0);
    }
    __syncwarp();
  }

  // ----------------------------------------------------------- teardown --
  if (*abort_word != 0) {
    // Give copies and MMAs still in flight time to land before TMEM and
    // shared memory are released.
    const uint64_t start = ptx::global_timer_ns();
    while (ptx::global_timer_ns() - start < 200000) __nanosleep(1000);
  }
  ptx::tc_fence_before_sync();
  if constexpr (PAIR) {
    // Neither CTA may leave while its partner can still touch its shared
    // memory (remote arrives, the pair MMA reading both operand halves).
    ptx::cluster_sync();
  } else {
    __syncthreads();
  }
  ptx::tc_fence_after_sync();
  if (warp == 1) {
    if constexpr (PAIR) {
      ptx::tmem_dealloc_pair(tmem_base, Cfg::kTmemCols);
    } else {
      ptx::tmem_dealloc(tmem_base, Cfg::kTmemCols);
    }
  }
  if (tracing && threadIdx.x == 0) {
    p.trace[blockIdx.x * kTraceWords + 9] = static_cast<uint64_t>(clock64() - kernel_t0);
  }
  if (threadIdx.x == 0 && leader) {
    if (p.cta_tiles != nullptr) p.cta_tiles[unit] = misc->tiles_done;
    if (p.sched_mode == kSchedQueue) {
      // The last unit to leave rearms the queue for the next launch.
      __threadfence();
      const uint32_t exited = atomicAdd(&p.queue[2], 1u);
      if (exited + 1 == units) {
        p.queue[0] = 0;
        // (with a device-side tile total there is no singly-claimed tail: park the
        // tail counter at the capacity so that it never hands anything out)
        p.queue[1] = p.tile_count_dev != nullptr ? p.tile_count : main_end;
        p.queue[2] = 0;
        __threadfence();
      }
    }
  }
}

template <uint32_t TILE_N, bool PAIR, bool OUT_F32>
cudaError_t launch_impl(const GemmParams& params, uint32_t units, cudaStream_t stream) {
  using Cfg = Config<TILE_N, PAIR>;
  // The opt-in shared-memory size is a per-device function attribute.
  static bool configured[64] = {};
  int device = 0;
  cudaError_t err = cudaGetDevice(&device);
  if (err != cudaSuccess) return err;
  if (device < 0 || device >= 64 || !configured[device]) {
    err = cudaFuncSetAttribute(grouped_gemm_kernel<TILE_N, PAIR, OUT_F32>,
                               cudaFuncAttributeMaxDynamicSharedMemorySize,
                               static_cast<int>(Cfg::kDynamicSmem));
    if (err != cudaSuccess) return err;
    if (device >= 0 && device < 64) configured[device] = true;
  }
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(units * Cfg::kGroup);
  config.blockDim = dim3(kThreads);
  config.dynamicSmemBytes = Cfg::kDynamicSmem;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeClusterDimension;
  attribute[0].val.clusterDim.x = Cfg::kGroup;
  attribute[0].val.clusterDim.y = 1;
  attribute[0].val.clusterDim.z = 1;
  config.attrs = attribute;
  config.numAttrs = 1;
  err = cudaLaunchKernelEx(&config, grouped_gemm_kernel<TILE_N, PAIR, OUT_F32>, params);
  return err != cudaSuccess ? err : cudaPeekAtLastError();
}

}  // namespace

uint32_t gemm_smem_bytes(uint32_t tile_n, uint32_t cta_group) {
  if (cta_group == 2) return Config<256, true>::kDynamicSmem;
  if (tile_n == 64) return Config<64, false>::kDynamicSmem;
  return tile_n == 256 ? Config<256, false>::kDynamicSmem : Config<128, false>::kDynamicSmem;
}

uint32_t gemm_stage_count(uint32_t tile_n, uint32_t cta_group) {
  if (cta_group == 2) return Config<256, true>::kStages;
  if (tile_n == 64) return Config<64, false>::kStages;
  return tile_n == 256 ? Config<256, false>::kStages : Config<128, false>::kStages;
}

cudaError_t preload_gemm_kernels() {
  cudaError_t rc = preload_one(grouped_gemm_kernel<256, true, false>);
  if (rc == cudaSuccess) rc = preload_one(grouped_gemm_kernel<256, false, false>);
  if (rc == cudaSuccess) rc = preload_one(grouped_gemm_kernel<128, false, false>);
  if (rc == cudaSuccess) rc = preload_one(grouped_gemm_kernel<64, false, false>);
  if (rc == cudaSuccess) rc = preload_one(grouped_gemm_kernel<256, true, true>);
  if (rc == cudaSuccess) rc = preload_one(grouped_gemm_kernel<256, false, true>);
  return rc;
}

cudaError_t launch_grouped_gemm(const GemmParams& params, uint32_t tile_n,
                                uint32_t cta_group, bool out_f32, uint32_t units,
                                cudaStream_t stream) {
  if (units == 0) return cudaSuccess;
  if (out_f32) {
    if (cta_group == 2 && tile_n == 256) return launch_impl<256, true, true>(params, units, stream);
    if (cta_group == 1 && tile_n == 256) return launch_impl<256, false, true>(params, units, stream);
    return cudaErrorInvalidValue;
  }
  if (cta_group == 2 && tile_n == 256) return launch_impl<256, true, false>(params, units, stream);
  if (cta_group == 1 && tile_n == 256) return launch_impl<256, false, false>(params, units, stream);
  if (cta_group == 1 && tile_n == 128) return launch_impl<128, false, false>(params, units, stream);
  if (cta_group == 1 && tile_n == 64) return launch_impl<64, false, false>(params, units, stream);
  return cudaErrorInvalidValue;
}

}  // namespace bmoe
