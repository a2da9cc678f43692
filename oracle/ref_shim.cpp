// C entry points around the REFERENCE's own host sources, so that tests can
// call them through ctypes. TEST INFRASTRUCTURE ONLY.
//
// This file is compiled together with the reference's
//   src/workload/workload.cpp  and  src/scheduler/scheduler.cpp
// taken from where the reference checkout lies (never copied into this
// repository), against the reference's own headers; build_oracle.py holds the
// recipe and writes oracle/_ref/libref_sched.so.
#include <cstdint>
#include <cstring>
#include <exception>
#include <random>
#include <vector>

#include "blackwell_moe/scheduler/scheduler.cuh"
#include "blackwell_moe/workload.hpp"

namespace bm = blackwell_moe;

namespace {

bm::GemmShape shape_of(uint32_t n, uint32_t tile_m, uint32_t tile_n) {
  bm::GemmShape s;
  s.n = n;
  s.tile_m = tile_m;
  s.tile_n = tile_n;
  return s;
}

uint64_t copy_tiles(const std::vector<bm::ExpertTile>& tiles, void* out, uint64_t cap) {
  const uint64_t n = tiles.size() < cap ? tiles.size() : cap;
  if (n != 0) std::memcpy(out, tiles.data(), n * sizeof(bm::ExpertTile));
  return tiles.size();
}

}  // namespace

extern "C" {

// The reference's draw loop (src/workload/workload.cpp:100-113) over an explicit
// weight vector: the same two standard-library objects, nothing else. Pins the
// restated mt19937_64 / discrete_distribution on weight vectors that none of the
// reference's four families produces (zero weights at the back).
int ref_draw_counts(const double* weights, uint32_t experts, uint64_t total_tokens,
                    uint64_t seed, uint32_t* counts_out) {
  if (weights == nullptr || counts_out == nullptr || experts == 0) return -1;
  std::mt19937_64 engine(seed);
  std::discrete_distribution<std::uint32_t> pick(weights, weights + experts);
  std::memset(counts_out, 0, sizeof(uint32_t) * experts);
  for (uint64_t t = 0; t < total_tokens; ++t) counts_out[pick(engine)] += 1;
  return 0;
}

int ref_generate_counts(uint32_t experts, uint64_t total_tokens, uint32_t distribution,
                        uint64_t seed, double zipf_alpha, double heavy_fraction,
                        double heavy_share, double inactive_fraction,
                        uint32_t* counts_out) {
  try {
    bm::WorkloadConfig c;
    c.experts = experts;
    c.total_tokens = total_tokens;
    c.distribution = static_cast<bm::Distribution>(distribution);
    c.seed = seed;
    c.zipf_alpha = zipf_alpha;
    c.heavy_hitter_fraction = heavy_fraction;
    c.heavy_hitter_token_share = heavy_share;
    c.inactive_expert_fraction = inactive_fraction;
    const bm::Workload w = bm::generate_workload(c);
    std::memcpy(counts_out, w.tokens_per_expert.data(), sizeof(uint32_t) * experts);
    return 0;
  } catch (const std::exception&) {
    return -1;
  }
}

int ref_workload_metrics(const uint32_t* counts, uint32_t experts, uint32_t n,
                         uint32_t tile_m, uint32_t tile_n, double* out,
                         uint64_t* out_int) {
  try {
    const bm::WorkloadMetrics m = bm::compute_workload_metrics(
        std::vector<uint32_t>(counts, counts + experts), shape_of(n, tile_m, tile_n));
    out[0] = m.mean_tokens;
    out[1] = m.coefficient_of_variation;
    out[2] = m.max_over_mean;
    out[3] = m.inactive_expert_ratio;
    out[4] = m.small_m_expert_ratio;
    out[5] = m.tile_count_cv;
    out_int[0] = m.active_experts;
    out_int[1] = m.total_tiles;
    return 0;
  } catch (const std::exception&) {
    return -1;
  }
}

// order 0: build_expert_tiles; order 1: order_by_descending_expert_tiles.
uint64_t ref_build_tiles(const uint32_t* counts, uint32_t experts, uint32_t n,
                         uint32_t tile_m, uint32_t tile_n, uint32_t order, void* out,
                         uint64_t cap) {
  try {
    const std::vector<uint32_t> tokens(counts, counts + experts);
    const bm::GemmShape s = shape_of(n, tile_m, tile_n);
    return copy_tiles(order == 0 ? bm::build_expert_tiles(tokens, s)
                                 : bm::order_by_descending_expert_tiles(tokens, s),
                      out, cap);
  } catch (const std::exception&) {
    return UINT64_MAX;
  }
}

uint64_t ref_simulate(uint32_t scheduler, const uint32_t* counts, uint32_t experts,
                      uint32_t n, uint32_t tile_m, uint32_t tile_n, uint32_t cta_count,
                      void* tiles_out, uint64_t cap, uint64_t* cta_offsets,
                      uint64_t* ints, double* reals) {
  try {
    const bm::GemmShape s = shape_of(n, tile_m, tile_n);
    const bm::CtaAssignment a = bm::simulate_scheduler(
        static_cast<bm::SchedulerKind>(scheduler),
        std::vector<uint32_t>(counts, counts + experts), s, cta_count);
    std::vector<bm::ExpertTile> flat;
    uint64_t cursor = 0;
    for (std::size_t c = 0; c < a.cta_tiles.size(); ++c) {
      cta_offsets[c] = cursor;
      flat.insert(flat.end(), a.cta_tiles[c].begin(), a.cta_tiles[c].end());
      cursor += a.cta_tiles[c].size();
    }
    cta_offsets[a.cta_tiles.size()] = cursor;
    copy_tiles(flat, tiles_out, cap);
    const bm::ScheduleMetrics m = bm::compute_schedule_metrics(a, s);
    ints[0] = m.total_tiles;
    ints[1] = m.total_valid_elements;
    ints[2] = m.total_padded_elements;
    ints[3] = m.expert_switches;
    ints[4] = m.min_tiles_per_cta;
    ints[5] = m.max_tiles_per_cta;
    reals[0] = m.mean_cta_work;
    reals[1] = m.max_cta_work;
    reals[2] = m.cta_work_cv;
    reals[3] = m.tail_ratio;
    reals[4] = m.estimated_utilization;
    reals[5] = m.useful_work_ratio;
    return cursor;
  } catch (const std::exception&) {
    return UINT64_MAX;
  }
}

}  // extern "C"
