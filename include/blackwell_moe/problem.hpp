// Problem description for MoE grouped GEMM: routing families, the workload
// descriptor (per-expert token counts) and the GEMM/tile shape.
//
// Source-compatible with the reference interface
// include/blackwell_moe/problem.hpp:9-40 (same type names, member order,
// defaults and enumerator ordinals), so reference callers compile unchanged.
#pragma once

#include <cstdint>
#include <string>
#include <vector>

namespace blackwell_moe {

// Routing family used by generate_workload(). Ordinals are part of the ABI
// (they are passed through the C interface as plain integers).
enum class Distribution {
  kUniform,      // 0: every expert equally likely
  kHeavyHitter,  // 1: a leading fraction of experts takes a fixed token share
  kSparse,       // 2: a leading fraction of experts receives nothing
  kZipf,         // 3: weight 1/(rank+1)^alpha
  // Appended (no reference counterpart): the two families above combined. The
  // first ceil(E * heavy_hitter_fraction) experts share heavy_hitter_token_share,
  // the LAST floor(E * inactive_expert_fraction) experts receive nothing, the
  // experts in between share the rest evenly. Decode-shaped routing with a hot
  // set and an idle set uses it.
  kHeavySparse,  // 4
};

std::string to_string(Distribution distribution);
// Accepts "uniform", "heavy_hitter" (alias "heavy"), "sparse", "zipf" and
// "heavy_sparse";
// anything else throws std::invalid_argument.
Distribution parse_distribution(const std::string& value);

struct WorkloadConfig {
  std::uint32_t experts = 64;
  // Number of (token, expert) assignments drawn, i.e. tokens * top_k.
  std::uint64_t total_tokens = 4096;
  Distribution distribution = Distribution::kUniform;
  std::uint64_t seed = 2026;
  double zipf_alpha = 1.2;
  double heavy_hitter_fraction = 0.1;
  double heavy_hitter_token_share = 0.8;
  double inactive_expert_fraction = 0.5;
};

// The workload descriptor: one routed-row count per expert.
struct Workload {
  WorkloadConfig config;
  std::vector<std::uint32_t> tokens_per_expert;
};

// Per-expert GEMM is D[M_e, n] = A[M_e, k] * B[n, k]^T; output tiles are
// tile_m x tile_n.
struct GemmShape {
  std::uint32_t n = 7168;
  std::uint32_t k = 2048;
  std::uint32_t tile_m = 128;
  std::uint32_t tile_n = 128;
};

}  // namespace blackwell_moe
