// The unit of GPU work: one output tile of one expert.
//
// Record layout is fixed (five 32-bit words, 20 bytes) and identical to the
// reference record include/blackwell_moe/work_tile.cuh:13-21; the device
// worklist builder emits exactly these bytes and the grouped-GEMM kernel
// consumes them.
#pragma once

#include <cstdint>

#if defined(__CUDACC__)
#define BMOE_TILE_FN __host__ __device__ inline
#else
#define BMOE_TILE_FN inline
#endif

namespace blackwell_moe {

struct ExpertTile {
  std::uint32_t expert_id;
  std::uint32_t tile_m;   // tile index along the expert's rows (not a row offset)
  std::uint32_t tile_n;   // tile index along the output columns
  std::uint32_t valid_m;  // rows of this tile that exist (< tile_m on the ragged edge)
  std::uint32_t valid_n;  // columns of this tile that exist
};

static_assert(sizeof(ExpertTile) == 20, "ExpertTile is a packed 20-byte record");

BMOE_TILE_FN bool operator==(const ExpertTile& a, const ExpertTile& b) {
  return a.expert_id == b.expert_id && a.tile_m == b.tile_m &&
         a.tile_n == b.tile_n && a.valid_m == b.valid_m &&
         a.valid_n == b.valid_n;
}

BMOE_TILE_FN bool operator!=(const ExpertTile& a, const ExpertTile& b) {
  return !(a == b);
}

// Number of logically valid output elements in the tile.
BMOE_TILE_FN std::uint64_t valid_output_elements(const ExpertTile& tile) {
  return static_cast<std::uint64_t>(tile.valid_m) * tile.valid_n;
}

}  // namespace blackwell_moe

#undef BMOE_TILE_FN
