// Expert -> rank placement for the expert-parallel layer: balance the number of
// GEMM tiles per rank. Deterministic longest-processing-time rule: experts in
// (more tiles first, lower id first) order, each to the rank with the fewest
// tiles so far (lowest rank on ties), optionally capped in experts per rank.
// The reference has no expert-parallel code (agent/search_space.yaml:10-13);
// tile counts use the same formula as its scheduler (src/scheduler/scheduler.cpp:44-47).
#include <algorithm>
#include <cstdint>
#include <numeric>
#include <vector>

#include "bmoe_b200.h"

extern "C" int bmoe_ep_place_experts(const uint32_t* global_counts, uint32_t experts,
                                     uint32_t ranks, uint32_t n, uint32_t tile_m,
                                     uint32_t tile_n, uint32_t max_experts_per_rank,
                                     uint32_t* owner_out, uint64_t* rank_tiles_out) {
  if (global_counts == nullptr || owner_out == nullptr || experts == 0 || ranks == 0 ||
      tile_m == 0 || tile_n == 0) {
    return BMOE_INVALID_ARGUMENT;
  }
  if (max_experts_per_rank != 0 &&
      static_cast<uint64_t>(max_experts_per_rank) * ranks < experts) {
    return BMOE_INVALID_ARGUMENT;
  }
  const uint64_t n_tiles = (static_cast<uint64_t>(n) + tile_n - 1) / tile_n;
  std::vector<uint64_t> tiles(experts);
  for (uint32_t e = 0; e < experts; ++e) {
    tiles[e] = ((static_cast<uint64_t>(global_counts[e]) + tile_m - 1) / tile_m) * n_tiles;
  }
  std::vector<uint32_t> order(experts);
  std::iota(order.begin(), order.end(), 0u);
  std::stable_sort(order.begin(), order.end(),
                   [&tiles](uint32_t a, uint32_t b) { return tiles[a] > tiles[b]; });
  std::vector<uint64_t> load(ranks, 0);
  std::vector<uint32_t> held(ranks, 0);
  for (uint32_t e : order) {
    uint32_t best = ranks;
    for (uint32_t r = 0; r < ranks; ++r) {
      if (max_experts_per_rank != 0 && held[r] >= max_experts_per_rank) continue;
      if (best == ranks || load[r] < load[best]) best = r;
    }
    owner_out[e] = best;
    load[best] += tiles[e];
    held[best] += 1;
  }
  if (rank_tiles_out != nullptr) {
    for (uint32_t r = 0; r < ranks; ++r) rank_tiles_out[r] = load[r];
  }
  return BMOE_OK;
}
