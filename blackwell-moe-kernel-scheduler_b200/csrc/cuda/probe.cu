// Scheduler probe: the static grid-stride and the atomic-queue persistent loops
// over integer stand-in work, with device counters that prove every tile ran
// exactly once and show how much work each CTA really took.
//
// Same observables and the same per-tile checksum as the reference probe
// (src/kernels/scheduler_probe.cu:26-101): every one of 256 threads hashes
// (expert, tile_m, tile_n, thread) for max(1, work_scale * ceil(valid/4096))
// rounds of the splitmix64 finaliser and the block XOR of the results is the
// tile's checksum.
#include <cuda_runtime.h>

#include <cstdint>

#include "blackwell_moe/scheduler/dynamic_queue.cuh"
#include "bmoe_b200.h"
#include "preload.cuh"

namespace bmoe {

namespace {

constexpr uint32_t kProbeThreads = 256;
constexpr uint32_t kProbeWarps = kProbeThreads / 32;

__device__ __forceinline__ uint64_t splitmix_finalise(uint64_t x) {
  x ^= x >> 30;
  x *= 0xbf58476d1ce4e5b9ull;
  x ^= x >> 27;
  x *= 0x94d049bb133111ebull;
  x ^= x >> 31;
  return x;
}

struct CtaTally {
  uint32_t tiles = 0;
  uint64_t valid = 0;
};

// Whole block: stand-in work for one tile, then thread 0 records the visit.
__device__ void visit_tile(const bmoe_probe_args& a, uint32_t tile_id,
                           uint64_t* warp_xor, CtaTally& tally) {
  const bmoe_tile t = a.tiles[tile_id];
  const uint64_t valid = static_cast<uint64_t>(t.valid_m) * t.valid_n;
  uint32_t rounds = a.work_scale * static_cast<uint32_t>((valid + 4095) / 4096);
  if (rounds == 0) rounds = 1;

  uint64_t h = (static_cast<uint64_t>(t.expert_id) << 48) ^
               (static_cast<uint64_t>(t.tile_m) << 32) ^
               (static_cast<uint64_t>(t.tile_n) << 16) ^ threadIdx.x;
  for (uint32_t r = 0; r < rounds; ++r) {
    h = splitmix_finalise(h + r + 0x9e3779b97f4a7c15ull);
  }
#pragma unroll
  for (uint32_t d = 16; d > 0; d >>= 1) {
    h ^= __shfl_xor_sync(0xffffffffu, h, d);
  }
  if ((threadIdx.x & 31) == 0) warp_xor[threadIdx.x >> 5] = h;
  __syncthreads();
  if (threadIdx.x == 0) {
    uint64_t all = 0;
    for (uint32_t w = 0; w < kProbeWarps; ++w) all ^= warp_xor[w];
    atomicAdd(a.tile_visits + tile_id, 1u);
    a.tile_checksums[tile_id] = all;
    tally.tiles += 1;
    tally.valid += valid;
  }
  __syncthreads();
}

__device__ void write_tally(const bmoe_probe_args& a, const CtaTally& tally) {
  if (threadIdx.x == 0) {
    a.cta_tile_counts[blockIdx.x] = tally.tiles;
    a.cta_valid_elements[blockIdx.x] = tally.valid;
  }
}

__global__ void __launch_bounds__(kProbeThreads)
probe_static_kernel(bmoe_probe_args a) {
  __shared__ uint64_t warp_xor[kProbeWarps];
  CtaTally tally;
  for (uint32_t t = blockIdx.x; t < a.tile_count; t += gridDim.x) {
    visit_tile(a, t, warp_xor, tally);
  }
  write_tally(a, tally);
}

__global__ void __launch_bounds__(kProbeThreads)
probe_queue_kernel(bmoe_probe_args a) {
  __shared__ uint64_t warp_xor[kProbeWarps];
  __shared__ uint32_t claim_begin;
  CtaTally tally;
  blackwell_moe::DynamicQueueState queue;
  queue.next_tile = a.next_tile;
  queue.tile_count = a.tile_count;
  queue.claim_size = a.claim_size;
  for (;;) {
    if (threadIdx.x == 0) claim_begin = blackwell_moe::claim_dynamic_tiles(queue);
    __syncthreads();
    const uint32_t begin = claim_begin;
    if (begin >= queue.tile_count) break;
    const uint32_t end = min(begin + queue.claim_size, queue.tile_count);
    for (uint32_t t = begin; t < end; ++t) visit_tile(a, t, warp_xor, tally);
    // visit_tile ends with a block barrier, so claim_begin may be rewritten.
  }
  write_tally(a, tally);
}

}  // namespace

}  // namespace bmoe

extern "C" {

int bmoe_probe_launch(uint32_t scheduler, const bmoe_probe_args* args) {
  if (args == nullptr) return BMOE_INVALID_ARGUMENT;
  const bmoe_probe_args& a = *args;
  const bool queue = scheduler == 1;
  if (scheduler > 1 || a.tiles == nullptr || a.tile_count == 0 || a.cta_count == 0 ||
      a.claim_size == 0 || a.work_scale == 0 || a.tile_visits == nullptr ||
      a.tile_checksums == nullptr || a.cta_tile_counts == nullptr ||
      a.cta_valid_elements == nullptr || (queue && a.next_tile == nullptr)) {
    return BMOE_INVALID_ARGUMENT;
  }
  cudaStream_t stream = static_cast<cudaStream_t>(a.stream);
  if (queue) {
    bmoe::probe_queue_kernel<<<a.cta_count, bmoe::kProbeThreads, 0, stream>>>(a);
  } else {
    bmoe::probe_static_kernel<<<a.cta_count, bmoe::kProbeThreads, 0, stream>>>(a);
  }
  return cudaPeekAtLastError() == cudaSuccess ? BMOE_OK : BMOE_CUDA_ERROR;
}

const char* bmoe_probe_scheduler_name(uint32_t scheduler) {
  switch (scheduler) {
    case 0: return "static_persistent_round_robin";
    case 1: return "dynamic_global_queue";
  }
  return "unknown";
}

}  // extern "C"

namespace bmoe {
cudaError_t preload_probe_kernels() {
  cudaError_t rc = preload_one(probe_static_kernel);
  if (rc == cudaSuccess) rc = preload_one(probe_queue_kernel);
  return rc;
}
}  // namespace bmoe
