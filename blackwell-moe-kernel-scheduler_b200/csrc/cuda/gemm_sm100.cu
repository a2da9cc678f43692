// Persistent, warp-specialised BF16 grouped GEMM for sm_100a.
//
// One CTA (256 threads) per SM walks a device worklist of 20-byte tile records
// and computes, per record, a 128 x TILE_N block of
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

#include <cuda_runtime.h>

#include "ptx_sm100.cuh"

namespace bmoe {

namespace {

constexpr uint32_t kThreads = 256;
constexpr uint32_t kTileM = 128;
constexpr uint32_t kBlockK = 64;                        // BF16 elements per k-block (128 B)
constexpr uint32_t kABytes = kTileM * kBlockK * 2;      // 16 KiB
constexpr uint32_t kSchedSlots = 4;
constexpr uint32_t kEpiWarps = 4;
constexpr uint32_t kStoreCols = 64;                     // columns per TMA store box
constexpr uint32_t kStoreRows = 32;                     // rows per epilogue warp
constexpr uint32_t kStoreBytes = kStoreRows * kStoreCols * 2;  // 4 KiB
constexpr uint32_t kStagingBytes = kEpiWarps * 2 * kStoreBytes;
constexpr int32_t kSentinel = -1;

template <uint32_t TILE_N>
struct Config {
  static constexpr uint32_t kStages = TILE_N == 256 ? 4 : 6;
  static constexpr uint32_t kBBytes = TILE_N * kBlockK * 2;
  static constexpr uint32_t kStageBytes = kABytes + kBBytes;
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

template <uint32_t TILE_N>
__global__ void __launch_bounds__(kThreads, 1)
grouped_gemm_kernel(const __grid_constant__ GemmParams p) {
  using Cfg = Config<TILE_N>;
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

  // ------------------------------------------------------------- set-up --
  if (threadIdx.x == 0) {
    for (uint32_t s = 0; s < Cfg::kStages; ++s) {
      ptx::mbar_init(bar_full(s), 1);
      ptx::mbar_init(bar_empty(s), 1);
    }
    for (uint32_t b = 0; b < 2; ++b) {
      ptx::mbar_init(bar_tmem_full(b), 1);
      ptx::mbar_init(bar_tmem_empty(b), kEpiWarps);
    }
    for (uint32_t s = 0; s < kSchedSlots; ++s) {
      ptx::mbar_init(bar_sched_full(s), 1);
      ptx::mbar_init(bar_sched_empty(s), 2 + kEpiWarps);  // producer, MMA, 4 epilogue warps
    }
    ptx::mbar_init(bar_clc, 1);
    misc->abort_word = 0;
    misc->producer_reads = 0;
    misc->tiles_done = 0;
    ptx::fence_barrier_init();
  }
  if (warp == 1) {
    ptx::tmem_alloc(base + Cfg::kOffMisc, Cfg::kTmemCols);  // -> misc->tmem_base
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = misc->tmem_base;

  // ---------------------------------------------------------- scheduler --
  if (warp == 2) {
    if (lane == 0) {
      uint32_t published = 0;
      bool alive = true;
      // Publishes one decoded record (or the sentinel) to the next ring slot.
      auto publish = [&](int32_t tile_index) -> bool {
        const uint32_t slot = published % kSchedSlots;
        const uint32_t round = (published / kSchedSlots) & 1u;
        if (!ptx::mbar_wait(bar_sched_empty(slot), round ^ 1u, abort_word, budget)) {
          report(p, kSiteSchedSlot, 0, static_cast<uint32_t>(tile_index), slot, published);
          return false;
        }
        volatile TileInfo* info = &slots[slot];
        info->tile = tile_index;
        if (tile_index != kSentinel) {
          const bmoe_tile rec = p.tiles[tile_index];
          info->expert = rec.expert_id;
          info->row0 = rec.tile_m * kTileM;
          info->col0 = rec.tile_n * TILE_N;
          info->valid_m = rec.valid_m;
          info->valid_n = rec.valid_n;
        }
        ptx::mbar_arrive(bar_sched_full(slot));
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
        for (uint32_t t = blockIdx.x; alive && t < p.tile_count; t += gridDim.x) {
          alive = publish(static_cast<int32_t>(t));
        }
      } else if (p.sched_mode == kSchedQueue) {
        // Main part: chunks of claim_size below main_end.
        while (alive) {
          if (!pace()) { alive = false; break; }
          const uint32_t begin = atomicAdd(&p.queue[0], p.claim_size);
          if (begin >= p.main_end) break;
          const uint32_t end = min(begin + p.claim_size, p.main_end);
          for (uint32_t t = begin; alive && t < end; ++t) {
            if (t != begin && !pace()) { alive = false; break; }
            alive = publish(static_cast<int32_t>(t));
          }
        }
        // Tail part: single tiles from the second counter.
        while (alive) {
          if (!pace()) { alive = false; break; }
          const uint32_t t = atomicAdd(&p.queue[1], 1u);
          if (t >= p.tile_count) break;
          alive = publish(static_cast<int32_t>(t));
        }
      } else {  // kSchedClc
        uint32_t clc_round = 0;
        uint32_t t = blockIdx.x;
        if (t < p.tile_count) alive = publish(static_cast<int32_t>(t));
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
          if (!got) break;  // no pending CTA left; must not ask again
          t = stolen;
          if (t < p.tile_count) alive = publish(static_cast<int32_t>(t));
        }
      }
      if (alive) publish(kSentinel);
    }
    __syncwarp();
  }

  // ----------------------------------------------------------- producer --
  else if (warp == 0) {
    if (lane == 0) {
      uint32_t reads = 0;
      uint32_t stage = 0, stage_round = 0;
      uint32_t last_expert = 0xffffffffu;
      while (true) {
        const uint32_t slot = reads % kSchedSlots;
        const uint32_t round = (reads / kSchedSlots) & 1u;
        if (!ptx::mbar_wait(bar_sched_full(slot), round, abort_word, budget)) {
          report(p, kSiteProducerInfo, 1, reads, slot, 0);
          break;
        }
        const int32_t tile = slots[slot].tile;
        const uint32_t expert = slots[slot].expert;
        const uint32_t row0 = slots[slot].row0;
        const uint32_t col0 = slots[slot].col0;
        ptx::mbar_arrive(bar_sched_empty(slot));
        ++reads;
        misc->producer_reads = reads;
        if (tile == kSentinel) break;

        const CUtensorMap* const map_a = p.tmap_a + expert;
        const CUtensorMap* const map_b = p.tmap_b + expert;
        if (expert != last_expert) {
          ptx::tensormap_acquire(map_a);
          ptx::tensormap_acquire(map_b);
          last_expert = expert;
        }
        bool ok = true;
        for (uint32_t kb = 0; kb < p.k_blocks; ++kb) {
          if (!ptx::mbar_wait(bar_empty(stage), stage_round ^ 1u, abort_word, budget)) {
            report(p, kSiteProducerStage, 1, static_cast<uint32_t>(tile), stage, kb);
            ok = false;
            break;
          }
          ptx::mbar_arrive_expect_tx(bar_full(stage), Cfg::kStageBytes);
          ptx::tma_load_2d(base + Cfg::kOffA + stage * kABytes, map_a, bar_full(stage),
                           static_cast<int32_t>(kb * kBlockK), static_cast<int32_t>(row0));
          ptx::tma_load_2d(base + Cfg::kOffB + stage * Cfg::kBBytes, map_b, bar_full(stage),
                           static_cast<int32_t>(kb * kBlockK), static_cast<int32_t>(col0));
          if (++stage == Cfg::kStages) { stage = 0; stage_round ^= 1u; }
        }
        if (!ok) break;
      }
    }
    __syncwarp();
  }

  // ---------------------------------------------------------------- MMA --
  else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = ptx::make_bf16_idesc(kTileM, TILE_N);
      uint32_t reads = 0;
      uint32_t stage = 0, stage_round = 0;
      uint32_t buf = 0, buf_round = 0;
      while (true) {
        const uint32_t slot = reads % kSchedSlots;
        const uint32_t round = (reads / kSchedSlots) & 1u;
        if (!ptx::mbar_wait(bar_sched_full(slot), round, abort_word, budget)) {
          report(p, kSiteMmaInfo, 2, reads, slot, 0);
          break;
        }
        const int32_t tile = slots[slot].tile;
        ptx::mbar_arrive(bar_sched_empty(slot));
        ++reads;
        if (tile == kSentinel) break;

        // The epilogue must have drained this accumulator buffer.
        if (!ptx::mbar_wait(bar_tmem_empty(buf), buf_round ^ 1u, abort_word, budget)) {
          report(p, kSiteMmaAccum, 2, static_cast<uint32_t>(tile), buf, 0);
          break;
        }
        ptx::tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + buf * TILE_N;
        bool ok = true;
        for (uint32_t kb = 0; kb < p.k_blocks; ++kb) {
          if (!ptx::mbar_wait(bar_full(stage), stage_round, abort_word, budget)) {
            report(p, kSiteMmaStage, 2, static_cast<uint32_t>(tile), stage, kb);
            ok = false;
            break;
          }
          ptx::tc_fence_after_sync();
          const uint64_t a_desc =
              ptx::make_kmajor_sw128_desc(base + Cfg::kOffA + stage * kABytes);
          const uint64_t b_desc =
              ptx::make_kmajor_sw128_desc(base + Cfg::kOffB + stage * Cfg::kBBytes);
#pragma unroll
          for (uint32_t ks = 0; ks < kBlockK / 16; ++ks) {
            // 16 BF16 = 32 bytes along k inside the 128-byte swizzle row.
            ptx::umma_bf16_ss(d_tmem, a_desc + 2 * ks, b_desc + 2 * ks, idesc,
                              (kb | ks) != 0 ? 1u : 0u);
          }
          ptx::umma_commit(bar_empty(stage));  // stage reusable once these MMAs retire
          if (++stage == Cfg::kStages) { stage = 0; stage_round ^= 1u; }
        }
        if (!ok) break;
        ptx::umma_commit(bar_tmem_full(buf));  // accumulator complete
        if (++buf == 2) { buf = 0; buf_round ^= 1u; }
      }
    }
    __syncwarp();
  }

  // ----------------------------------------------------------- epilogue --
  else if (warp >= 4) {
    const uint32_t quad = warp & 3u;  // TMEM lane quadrant this warp may read
    const uint32_t staging = base + Cfg::kOffStaging + quad * 2 * kStoreBytes;
    uint32_t reads = 0;
    uint32_t buf = 0, buf_round = 0;
    uint32_t sbuf = 0;
    uint32_t last_expert = 0xffffffffu;
    uint32_t tiles_done = 0;
    while (true) {
      const uint32_t slot = reads % kSchedSlots;
      const uint32_t round = (reads / kSchedSlots) & 1u;
      if (!ptx::mbar_wait(bar_sched_full(slot), round, abort_word, budget)) {
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
      if (lane == 0) ptx::mbar_arrive(bar_sched_empty(slot));
      ++reads;
      if (tile == kSentinel) break;

      if (!ptx::mbar_wait(bar_tmem_full(buf), buf_round, abort_word, budget)) {
        if (lane == 0 && quad == 0) {
          report(p, kSiteEpiAccum, 3, static_cast<uint32_t>(tile), buf, 0);
        }
        break;
      }
      ptx::tc_fence_after_sync();

      const CUtensorMap* const map_d = p.tmap_d + expert;
      if (lane == 0 && expert != last_expert) ptx::tensormap_acquire(map_d);
      last_expert = expert;

      const bool has_rows = quad * kStoreRows < valid_m;
      const uint32_t chunks = has_rows ? (valid_n + kStoreCols - 1) / kStoreCols : 0;
      const uint32_t lane_taddr = tmem_base + ((quad * 32u) << 16) + buf * TILE_N;
      for (uint32_t c = 0; c < chunks; ++c) {
        uint32_t lo[32], hi[32];
        ptx::tmem_load_32x32(lane_taddr + c * kStoreCols, lo);
        ptx::tmem_load_32x32(lane_taddr + c * kStoreCols + 32, hi);
        ptx::tmem_load_wait();
        if (c + 1 == chunks) {
          // All of this warp's accumulator rows are in registers: hand the
          // buffer back before the (slower) conversion and store.
          ptx::tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(bar_tmem_empty(buf));
        }
        // The store issued two chunks ago read from this staging buffer.
        if (lane == 0) ptx::tma_store_wait_read<1>();
        __syncwarp();
        const uint32_t row_smem = staging + sbuf * kStoreBytes + lane * 128u;
        const uint32_t sw = lane & 7u;
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
        ptx::fence_async_shared();
        __syncwarp();
        if (lane == 0) {
          ptx::tma_store_2d(map_d, staging + sbuf * kStoreBytes,
                            static_cast<int32_t>(col0 + c * kStoreCols),
                            static_cast<int32_t>(row0 + quad * kStoreRows));
          ptx::tma_store_commit();
        }
        sbuf ^= 1u;
      }
      if (chunks == 0) {
        // Nothing to read for this warp (rows beyond the ragged edge).
        ptx::tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(bar_tmem_empty(buf));
      }
      if (++buf == 2) { buf = 0; buf_round ^= 1u; }
      ++tiles_done;
      if (quad == 0 && lane == 0 && p.tile_visits != nullptr) {
        atomicAdd(&p.tile_visits[tile], 1u);
      }
    }
    if (lane == 0) ptx::tma_store_wait_all();
    if (quad == 0 && lane == 0) misc->tiles_done = tiles_done;
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
  __syncthreads();
  ptx::tc_fence_after_sync();
  if (warp == 1) {
    ptx::tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
  if (threadIdx.x == 0) {
    if (p.cta_tiles != nullptr) p.cta_tiles[blockIdx.x] = misc->tiles_done;
    if (p.sched_mode == kSchedQueue) {
      // The last CTA to leave rearms the queue for the next launch.
      __threadfence();
      const uint32_t exited = atomicAdd(&p.queue[2], 1u);
      if (exited + 1 == gridDim.x) {
        p.queue[0] = 0;
        p.queue[1] = p.main_end;
        p.queue[2] = 0;
        __threadfence();
      }
    }
  }
}

template <uint32_t TILE_N>
cudaError_t launch_impl(const GemmParams& params, uint32_t grid, cudaStream_t stream) {
  using Cfg = Config<TILE_N>;
  // The opt-in shared-memory size is a per-device function attribute.
  static bool configured[64] = {};
  int device = 0;
  cudaError_t err = cudaGetDevice(&device);
  if (err != cudaSuccess) return err;
  if (device < 0 || device >= 64 || !configured[device]) {
    err = cudaFuncSetAttribute(grouped_gemm_kernel<TILE_N>,
                               cudaFuncAttributeMaxDynamicSharedMemorySize,
                               static_cast<int>(Cfg::kDynamicSmem));
    if (err != cudaSuccess) return err;
    if (device >= 0 && device < 64) configured[device] = true;
  }
  grouped_gemm_kernel<TILE_N><<<grid, kThreads, Cfg::kDynamicSmem, stream>>>(params);
  return cudaPeekAtLastError();
}

}  // namespace

uint32_t gemm_smem_bytes(uint32_t tile_n) {
  return tile_n == 256 ? Config<256>::kDynamicSmem : Config<128>::kDynamicSmem;
}

uint32_t gemm_stage_count(uint32_t tile_n) {
  return tile_n == 256 ? Config<256>::kStages : Config<128>::kStages;
}

cudaError_t launch_grouped_gemm(const GemmParams& params, uint32_t tile_n,
                                uint32_t grid, cudaStream_t stream) {
  if (grid == 0) return cudaSuccess;
  if (tile_n == 256) return launch_impl<256>(params, grid, stream);
  if (tile_n == 128) return launch_impl<128>(params, grid, stream);
  return cudaErrorInvalidValue;
}

}  // namespace bmoe
