// Global atomic tile queue shared by the grouped-GEMM kernel and the
// scheduler probe (reference ABI:
// include/blackwell_moe/scheduler/dynamic_queue.cuh:10-24).
#pragma once

#include <cstdint>

namespace blackwell_moe {

// One 32-bit head counter in global memory. A claim advances it by claim_size
// and owns the half-open range [begin, min(begin + claim_size, tile_count)).
// A claim whose begin is >= tile_count means the queue is drained.
struct DynamicQueueState {
  std::uint32_t* next_tile = nullptr;
  std::uint32_t tile_count = 0;
  std::uint32_t claim_size = 1;
};

#if defined(__CUDACC__)
// Returns `begin` of the claimed range; the caller clamps the end.
__device__ __forceinline__ std::uint32_t claim_dynamic_tiles(
    const DynamicQueueState& queue) {
  return atomicAdd(queue.next_tile, queue.claim_size);
}
#endif

}  // namespace blackwell_moe
