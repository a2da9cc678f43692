// Routing features, threshold dispatch and scheduler claim-order models.
//
// Restates the reference's Python host logic in C++ with the same arithmetic
// (including CPython 3.12's compensated float sum), so the doubles agree bit
// for bit with the reference run under CPython >= 3.12 on the same libm:
//   routing_features   python/blackwell_moe_tirx/dispatch.py:42-83
//   select_kernel      python/blackwell_moe_tirx/dispatch.py:86-114
//   claim models       python/blackwell_moe_tirx/config.py:222-267
//   launch contracts   python/blackwell_moe_tirx/kernels/registry.py:31-42
#include "blackwell_moe/dispatch.hpp"

#include <algorithm>
#include <cmath>
#include <stdexcept>

namespace blackwell_moe {

namespace {

// Float accumulation as CPython >= 3.12 `sum()` performs it (Neumaier's
// compensated summation): the reference's variance sums go through it.
class PySum {
 public:
  void add(double x) {
    const double t = sum_ + x;
    comp_ += std::fabs(sum_) >= std::fabs(x) ? (sum_ - t) + x : (x - t) + sum_;
    sum_ = t;
  }
  double result() const {
    return (comp_ != 0.0 && std::isfinite(comp_)) ? sum_ + comp_ : sum_;
  }

 private:
  double sum_ = 0.0;
  double comp_ = 0.0;
};

// Mean, population CV and max/mean of a list of non-negative integers.
struct Spread {
  double mean = 0.0;
  double cv = 0.0;
  double max_over_mean = 0.0;
};

Spread spread_of(const std::vector<std::uint64_t>& xs) {
  Spread s;
  if (xs.empty()) return s;
  std::uint64_t total = 0;
  std::uint64_t largest = 0;
  for (std::uint64_t x : xs) {
    total += x;
    largest = std::max(largest, x);
  }
  s.mean = static_cast<double>(total) / static_cast<double>(xs.size());
  if (s.mean == 0.0) return s;
  PySum ss;
  for (std::uint64_t x : xs) {
    ss.add(std::pow(static_cast<double>(x) - s.mean, 2.0));
  }
  s.cv = std::sqrt(ss.result() / static_cast<double>(xs.size())) / s.mean;
  s.max_over_mean = static_cast<double>(largest) / s.mean;
  return s;
}

}  // namespace

const char* launch_variant_name(LaunchVariant variant) {
  switch (variant) {
    case LaunchVariant::kNonPersistent: return "v0_nonpersistent";
    case LaunchVariant::kStaticWs: return "v1_static_ws";
    case LaunchVariant::kDynamicClaim1: return "v2_dynamic";
    case LaunchVariant::kChunked: return "v3_chunked";
    case LaunchVariant::kHybrid: return "v4_hybrid";
    case LaunchVariant::kClc: return "v5_clc";
  }
  return "unknown";
}

RoutingFeatures routing_features(
    const std::vector<std::uint32_t>& tokens_per_expert,
    const GemmShape& shape,
    std::uint32_t cta_count) {
  if (shape.tile_m == 0 || shape.tile_n == 0) {
    throw std::invalid_argument("tile dimensions must be positive");
  }
  if (cta_count == 0) throw std::invalid_argument("cta_count must be positive");

  RoutingFeatures f;
  const std::size_t experts = tokens_per_expert.size();
  std::vector<std::uint64_t> rows(tokens_per_expert.begin(),
                                  tokens_per_expert.end());
  const Spread row_spread = spread_of(rows);
  f.mean_m = row_spread.mean;
  f.cv_m = row_spread.cv;
  f.max_over_mean_m = row_spread.max_over_mean;

  std::size_t active = 0;
  std::size_t small = 0;
  std::uint64_t row_total = 0;
  for (std::uint32_t c : tokens_per_expert) {
    row_total += c;
    if (c > 0) {
      ++active;
      if (c <= shape.tile_m) ++small;
    }
  }
  if (experts != 0) {
    f.inactive_expert_ratio =
        1.0 - static_cast<double>(active) / static_cast<double>(experts);
  }
  if (active != 0) {
    f.small_m_expert_ratio =
        static_cast<double>(small) / static_cast<double>(active);
  }

  // Per-expert tile statistics use whole column tiles only (n / tile_n), the
  // tile total below counts the ragged column tile too.
  const std::uint64_t whole_n_tiles = shape.n / shape.tile_n;
  const std::uint64_t all_n_tiles = (shape.n + shape.tile_n - 1) / shape.tile_n;
  std::vector<std::uint64_t> tiles(experts);
  std::uint64_t m_tile_total = 0;
  for (std::size_t e = 0; e < experts; ++e) {
    const std::uint64_t m_tiles =
        (static_cast<std::uint64_t>(tokens_per_expert[e]) + shape.tile_m - 1) /
        shape.tile_m;
    tiles[e] = m_tiles * whole_n_tiles;
    m_tile_total += m_tiles;
  }
  const Spread tile_spread = spread_of(tiles);
  f.expert_tile_cv = tile_spread.cv;
  f.max_expert_tiles_over_mean = tile_spread.max_over_mean;

  f.active_tiles = m_tile_total * all_n_tiles;
  f.tiles_per_cta =
      static_cast<double>(f.active_tiles) / static_cast<double>(cta_count);
  // logical / padded FLOPs; the common factor 2*k cancels.
  const std::uint64_t padded = f.active_tiles *
                               static_cast<std::uint64_t>(shape.tile_m) *
                               shape.tile_n;
  f.useful_work_ratio =
      padded == 0 ? 1.0
                  : static_cast<double>(row_total * shape.n) /
                        static_cast<double>(padded);
  return f;
}

LaunchVariant select_launch_variant(const RoutingFeatures& f,
                                    const DispatchThresholds& t) {
  if (f.tiles_per_cta <= t.nonpersistent_tiles_per_cta) {
    return LaunchVariant::kNonPersistent;
  }
  if (f.cv_m <= t.static_cv_m) return LaunchVariant::kStaticWs;
  if (f.tiles_per_cta < t.dynamic_min_tiles_per_cta) {
    return LaunchVariant::kStaticWs;
  }
  const bool deep_queue = f.tiles_per_cta >= t.chunked_min_tiles_per_cta;
  if (deep_queue && (f.cv_m >= t.high_skew_cv_m ||
                     f.inactive_expert_ratio >= t.sparse_expert_ratio)) {
    return LaunchVariant::kHybrid;
  }
  if (deep_queue) return LaunchVariant::kChunked;
  return LaunchVariant::kDynamicClaim1;
}

LaunchVariant select_launch_variant_fitted(const RoutingFeatures& f,
                                           const FittedDispatch& rule) {
  if (f.tiles_per_cta <= rule.nonpersistent_tiles_per_cta) {
    return LaunchVariant::kNonPersistent;
  }
  const double active_share = 1.0 - f.inactive_expert_ratio;
  const double mean_active_rows = active_share > 0.0 ? f.mean_m / active_share : 0.0;
  if (mean_active_rows <= rule.weight_stream_mean_rows) return LaunchVariant::kStaticWs;
  return LaunchVariant::kClc;
}

LaunchConfig resolve_launch_config(LaunchVariant variant,
                                   const DispatchSpec& spec) {
  LaunchConfig cfg;
  cfg.variant = variant;
  switch (variant) {
    case LaunchVariant::kNonPersistent:
      cfg.scheduler = SchedulerKind::kExpertOrder;
      cfg.one_cta_per_tile = true;
      break;
    case LaunchVariant::kStaticWs:
      cfg.scheduler = SchedulerKind::kStaticPersistent;
      break;
    case LaunchVariant::kDynamicClaim1:
      cfg.scheduler = SchedulerKind::kDynamicQueue;
      cfg.claim_size = 1;
      break;
    case LaunchVariant::kChunked:
      cfg.scheduler = SchedulerKind::kDynamicQueue;
      cfg.claim_size = spec.claim_size;
      break;
    case LaunchVariant::kHybrid:
      cfg.scheduler = SchedulerKind::kDynamicQueue;
      cfg.claim_size = spec.hybrid_main_claim_size;
      cfg.hybrid_tail_tiles = spec.hybrid_tail_tiles;
      break;
    case LaunchVariant::kClc:
      cfg.scheduler = SchedulerKind::kClc;
      cfg.one_cta_per_tile = true;
      break;
  }
  return cfg;
}

std::vector<std::vector<std::uint32_t>> static_cta_assignments(
    std::uint32_t tile_count, std::uint32_t cta_count) {
  if (cta_count == 0) throw std::invalid_argument("cta_count must be positive");
  std::vector<std::vector<std::uint32_t>> per_cta(cta_count);
  for (std::uint32_t t = 0; t < tile_count; ++t) {
    per_cta[t % cta_count].push_back(t);
  }
  return per_cta;
}

std::vector<std::vector<std::uint32_t>> chunked_claims(
    std::uint32_t tile_count, std::uint32_t claim_size) {
  if (claim_size == 0) throw std::invalid_argument("claim_size must be positive");
  std::vector<std::vector<std::uint32_t>> batches;
  for (std::uint64_t begin = 0; begin < tile_count; begin += claim_size) {
    const std::uint64_t end =
        std::min<std::uint64_t>(begin + claim_size, tile_count);
    std::vector<std::uint32_t> batch;
    for (std::uint64_t t = begin; t < end; ++t) {
      batch.push_back(static_cast<std::uint32_t>(t));
    }
    batches.push_back(std::move(batch));
  }
  return batches;
}

std::vector<std::vector<std::uint32_t>> hybrid_claims(
    std::uint32_t tile_count, std::uint32_t main_claim_size,
    std::uint32_t tail_tiles) {
  if (main_claim_size == 0) {
    throw std::invalid_argument("main_claim_size must be positive");
  }
  const std::uint32_t tail_begin = tile_count - std::min(tile_count, tail_tiles);
  std::vector<std::vector<std::uint32_t>> batches =
      chunked_claims(tail_begin, main_claim_size);
  for (std::uint32_t t = tail_begin; t < tile_count; ++t) {
    batches.push_back(std::vector<std::uint32_t>{t});
  }
  return batches;
}

}  // namespace blackwell_moe
