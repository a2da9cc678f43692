// Workload generation and routing statistics.
//
// Source-compatible with the reference interface
// include/blackwell_moe/workload.hpp:10-27. generate_workload() reproduces the
// reference token counts draw for draw (std::mt19937_64 seeded with
// config.seed feeding std::discrete_distribution, src/workload/workload.cpp:100-113),
// which ties the exact counts to GNU libstdc++.
#pragma once

#include <cstdint>
#include <vector>

#include "blackwell_moe/problem.hpp"

namespace blackwell_moe {

struct WorkloadMetrics {
  double mean_tokens = 0.0;
  double coefficient_of_variation = 0.0;  // population CV of tokens per expert
  double max_over_mean = 0.0;
  double inactive_expert_ratio = 0.0;     // experts with zero tokens / experts
  double small_m_expert_ratio = 0.0;      // experts with 0 < tokens < tile_m / experts
  double tile_count_cv = 0.0;             // population CV of tiles per expert
  std::uint32_t active_experts = 0;
  std::uint64_t total_tiles = 0;
};

// Throws std::invalid_argument for experts == 0, zipf_alpha <= 0 or fractions
// outside [0, 1] (heavy_hitter_fraction must also be non-zero).
Workload generate_workload(const WorkloadConfig& config);

// Empty input yields a zero-initialised result; zero tile dimensions throw.
WorkloadMetrics compute_workload_metrics(
    const std::vector<std::uint32_t>& tokens_per_expert,
    const GemmShape& shape);

// Throws when the count vector length differs from config.experts or the
// counts do not add up to config.total_tokens.
void validate_workload(const Workload& workload);

}  // namespace blackwell_moe
