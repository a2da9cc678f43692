// Routed-token workload generator and routing statistics (host side).
//
// Behaviour follows src/workload/workload.cpp of the reference:
//   expert weights per routing family          workload.cpp:13-49
//     (+ kHeavySparse, the heavy-hitter and sparse rules combined; appended here)
//   config validation                          workload.cpp:64-76
//   generate_workload                          workload.cpp:100-113
//   validate_workload                          workload.cpp:115-125
//   compute_workload_metrics                   workload.cpp:127-172
// The draw sequence (std::mt19937_64 -> std::discrete_distribution) is what
// fixes the exact counts, so the same two standard-library objects are used.
#include "blackwell_moe/workload.hpp"

#include <algorithm>
#include <cmath>
#include <random>
#include <stdexcept>

namespace blackwell_moe {

namespace {

bool is_fraction(double x) { return x >= 0.0 && x <= 1.0; }

void check_config(const WorkloadConfig& cfg) {
  if (cfg.experts == 0) {
    throw std::invalid_argument("experts must be positive");
  }
  if (!(cfg.zipf_alpha > 0.0)) {
    throw std::invalid_argument("zipf_alpha must be positive");
  }
  const bool fractions_ok = is_fraction(cfg.heavy_hitter_fraction) &&
                            cfg.heavy_hitter_fraction != 0.0 &&
                            is_fraction(cfg.heavy_hitter_token_share) &&
                            is_fraction(cfg.inactive_expert_fraction);
  if (!fractions_ok) {
    throw std::invalid_argument("distribution fractions must be within [0, 1]");
  }
}

// Unnormalised selection weight of every expert.
std::vector<double> expert_weights(const WorkloadConfig& cfg) {
  const std::uint32_t e = cfg.experts;
  std::vector<double> w(e, 1.0);
  if (cfg.distribution == Distribution::kZipf) {
    for (std::uint32_t rank = 0; rank < e; ++rank) {
      w[rank] = 1.0 / std::pow(static_cast<double>(rank + 1), cfg.zipf_alpha);
    }
  } else if (cfg.distribution == Distribution::kHeavyHitter) {
    const std::uint32_t heavy = std::max<std::uint32_t>(
        1u, static_cast<std::uint32_t>(std::ceil(e * cfg.heavy_hitter_fraction)));
    const std::uint32_t light = e - heavy;
    const double heavy_w = cfg.heavy_hitter_token_share / heavy;
    const double light_w =
        light == 0 ? 0.0 : (1.0 - cfg.heavy_hitter_token_share) / light;
    for (std::uint32_t i = 0; i < e; ++i) w[i] = i < heavy ? heavy_w : light_w;
  } else if (cfg.distribution == Distribution::kSparse) {
    const std::uint32_t silent = std::min<std::uint32_t>(
        e - 1,
        static_cast<std::uint32_t>(std::floor(e * cfg.inactive_expert_fraction)));
    for (std::uint32_t i = 0; i < silent; ++i) w[i] = 0.0;
  } else if (cfg.distribution == Distribution::kHeavySparse) {
    // Hot set in front (the heavy-hitter rule), idle set at the back (the sparse
    // rule's count), the experts in between share what the hot set leaves.
    const std::uint32_t silent = std::min<std::uint32_t>(
        e - 1,
        static_cast<std::uint32_t>(std::floor(e * cfg.inactive_expert_fraction)));
    const std::uint32_t heavy = std::min<std::uint32_t>(
        e - silent,
        std::max<std::uint32_t>(
            1u, static_cast<std::uint32_t>(std::ceil(e * cfg.heavy_hitter_fraction))));
    const std::uint32_t light = e - silent - heavy;
    const double heavy_w =
        (light == 0 ? 1.0 : cfg.heavy_hitter_token_share) / heavy;
    const double light_w =
        light == 0 ? 0.0 : (1.0 - cfg.heavy_hitter_token_share) / light;
    for (std::uint32_t i = 0; i < e; ++i) {
      w[i] = i < heavy ? heavy_w : (i < heavy + light ? light_w : 0.0);
    }
  }
  return w;
}

// Population coefficient of variation; 0 for empty input or zero mean.
double population_cv(const std::vector<double>& xs) {
  if (xs.empty()) return 0.0;
  double total = 0.0;
  for (double x : xs) total += x;
  const double mean = total / xs.size();
  if (mean == 0.0) return 0.0;
  double ss = 0.0;
  for (double x : xs) {
    const double d = x - mean;
    ss += d * d;
  }
  return std::sqrt(ss / xs.size()) / mean;
}

}  // namespace

std::string to_string(Distribution distribution) {
  switch (distribution) {
    case Distribution::kUniform: return "uniform";
    case Distribution::kHeavyHitter: return "heavy_hitter";
    case Distribution::kSparse: return "sparse";
    case Distribution::kZipf: return "zipf";
    case Distribution::kHeavySparse: return "heavy_sparse";
  }
  throw std::invalid_argument("unknown distribution");
}

Distribution parse_distribution(const std::string& value) {
  static const struct { const char* name; Distribution d; } table[] = {
      {"uniform", Distribution::kUniform},
      {"heavy_hitter", Distribution::kHeavyHitter},
      {"heavy", Distribution::kHeavyHitter},
      {"sparse", Distribution::kSparse},
      {"zipf", Distribution::kZipf},
      {"heavy_sparse", Distribution::kHeavySparse},
  };
  for (const auto& row : table) {
    if (value == row.name) return row.d;
  }
  throw std::invalid_argument("unknown distribution: " + value);
}

Workload generate_workload(const WorkloadConfig& config) {
  check_config(config);
  const std::vector<double> weights = expert_weights(config);
  std::mt19937_64 engine(config.seed);
  std::discrete_distribution<std::uint32_t> pick(weights.begin(), weights.end());

  Workload out;
  out.config = config;
  out.tokens_per_expert.assign(config.experts, 0u);
  for (std::uint64_t draw = 0; draw < config.total_tokens; ++draw) {
    out.tokens_per_expert[pick(engine)] += 1;
  }
  validate_workload(out);
  return out;
}

void validate_workload(const Workload& workload) {
  if (workload.tokens_per_expert.size() != workload.config.experts) {
    throw std::invalid_argument("tokens_per_expert size does not match experts");
  }
  std::uint64_t sum = 0;
  for (std::uint32_t c : workload.tokens_per_expert) sum += c;
  if (sum != workload.config.total_tokens) {
    throw std::invalid_argument("tokens_per_expert does not conserve tokens");
  }
}

WorkloadMetrics compute_workload_metrics(
    const std::vector<std::uint32_t>& tokens_per_expert,
    const GemmShape& shape) {
  WorkloadMetrics m;
  if (tokens_per_expert.empty()) return m;
  if (shape.tile_m == 0 || shape.tile_n == 0) {
    throw std::invalid_argument("tile dimensions must be positive");
  }
  const std::size_t experts = tokens_per_expert.size();
  const std::uint32_t n_tiles = (shape.n + shape.tile_n - 1) / shape.tile_n;

  std::uint64_t token_sum = 0;
  std::uint32_t largest = 0;
  std::uint32_t silent = 0;
  std::uint32_t small = 0;
  std::vector<double> as_tokens(experts);
  std::vector<double> as_tiles(experts);
  for (std::size_t e = 0; e < experts; ++e) {
    const std::uint32_t c = tokens_per_expert[e];
    token_sum += c;
    largest = std::max(largest, c);
    if (c == 0) {
      ++silent;
    } else {
      ++m.active_experts;
      if (c < shape.tile_m) ++small;
    }
    const std::uint64_t m_tiles =
        c == 0 ? 0 : (c + shape.tile_m - 1) / shape.tile_m;
    const std::uint64_t tiles = m_tiles * n_tiles;
    m.total_tiles += tiles;
    as_tokens[e] = static_cast<double>(c);
    as_tiles[e] = static_cast<double>(tiles);
  }
  m.mean_tokens = static_cast<double>(token_sum) / experts;
  m.coefficient_of_variation = population_cv(as_tokens);
  m.tile_count_cv = population_cv(as_tiles);
  m.max_over_mean = m.mean_tokens == 0.0 ? 0.0 : largest / m.mean_tokens;
  m.inactive_expert_ratio = static_cast<double>(silent) / experts;
  m.small_m_expert_ratio = static_cast<double>(small) / experts;
  return m;
}

}  // namespace blackwell_moe
