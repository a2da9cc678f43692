// C interface, host-model half: plain-C access to the workload generator, the
// worklist / policy model and the dispatch rule (section 1 of bmoe_b200.h).
// Exceptions of the C++ layer become BMOE_INVALID_ARGUMENT.
#include <algorithm>
#include <cstring>
#include <limits>
#include <stdexcept>
#include <vector>

#include "blackwell_moe/dispatch.hpp"
#include "blackwell_moe/kernels/grouped_gemm.cuh"
#include "blackwell_moe/scheduler/scheduler.cuh"
#include "blackwell_moe/workload.hpp"
#include "bmoe_b200.h"

namespace bm = blackwell_moe;

namespace {

bm::GemmShape make_shape(uint32_t n, uint32_t tile_m, uint32_t tile_n) {
  bm::GemmShape s;
  s.n = n;
  s.tile_m = tile_m;
  s.tile_n = tile_n;
  return s;
}

std::vector<uint32_t> to_vector(const uint32_t* counts, uint32_t experts) {
  return std::vector<uint32_t>(counts, counts + experts);
}

// Re-walks an expert's tile grid with tile_m as the fast index.
void append_m_fastest(std::vector<bm::ExpertTile>& out, uint32_t expert,
                      uint32_t tokens, const bm::GemmShape& s) {
  if (tokens == 0) return;
  const uint32_t m_tiles = (tokens + s.tile_m - 1) / s.tile_m;
  const uint32_t n_tiles = (s.n + s.tile_n - 1) / s.tile_n;
  for (uint32_t tn = 0; tn < n_tiles; ++tn) {
    const uint32_t cols = std::min(s.tile_n, s.n - tn * s.tile_n);
    for (uint32_t tm = 0; tm < m_tiles; ++tm) {
      const uint32_t rows = std::min(s.tile_m, tokens - tm * s.tile_m);
      out.push_back(bm::ExpertTile{expert, tm, tn, rows, cols});
    }
  }
}

}  // namespace

extern "C" {

const char* bmoe_status_string(int status) {
  switch (status) {
    case BMOE_OK: return "success";
    case BMOE_INVALID_ARGUMENT: return "invalid argument";
    case BMOE_UNSUPPORTED_DATA_TYPE: return "unsupported data type";
    case BMOE_UNSUPPORTED_SCHEDULER: return "unsupported scheduler";
    case BMOE_UNSUPPORTED_DEVICE: return "unsupported device";
    case BMOE_CUDA_ERROR: return "CUDA error";
    case BMOE_BACKEND_ERROR: return "CUTLASS error";
    case BMOE_DEVICE_TIMEOUT: return "device wait timed out";
  }
  return "unknown status";
}

int bmoe_generate_workload(const bmoe_workload_config* config,
                           uint32_t* counts_out) {
  if (config == nullptr || counts_out == nullptr) return BMOE_INVALID_ARGUMENT;
  if (config->distribution > 4) return BMOE_INVALID_ARGUMENT;
  try {
    bm::WorkloadConfig c;
    c.experts = config->experts;
    c.total_tokens = config->total_tokens;
    c.distribution = static_cast<bm::Distribution>(config->distribution);
    c.seed = config->seed;
    c.zipf_alpha = config->zipf_alpha;
    c.heavy_hitter_fraction = config->heavy_hitter_fraction;
    c.heavy_hitter_token_share = config->heavy_hitter_token_share;
    c.inactive_expert_fraction = config->inactive_expert_fraction;
    const bm::Workload w = bm::generate_workload(c);
    std::memcpy(counts_out, w.tokens_per_expert.data(),
                sizeof(uint32_t) * w.tokens_per_expert.size());
    return BMOE_OK;
  } catch (const std::exception&) {
    return BMOE_INVALID_ARGUMENT;
  }
}

int bmoe_workload_metrics_compute(const uint32_t* counts, uint32_t experts,
                                  uint32_t n, uint32_t tile_m, uint32_t tile_n,
                                  bmoe_workload_metrics* out) {
  if (out == nullptr || (counts == nullptr && experts != 0)) {
    return BMOE_INVALID_ARGUMENT;
  }
  try {
    const bm::WorkloadMetrics m = bm::compute_workload_metrics(
        to_vector(counts, experts), make_shape(n, tile_m, tile_n));
    out->mean_tokens = m.mean_tokens;
    out->coefficient_of_variation = m.coefficient_of_variation;
    out->max_over_mean = m.max_over_mean;
    out->inactive_expert_ratio = m.inactive_expert_ratio;
    out->small_m_expert_ratio = m.small_m_expert_ratio;
    out->tile_count_cv = m.tile_count_cv;
    out->active_experts = m.active_experts;
    out->reserved = 0;
    out->total_tiles = m.total_tiles;
    return BMOE_OK;
  } catch (const std::exception&) {
    return BMOE_INVALID_ARGUMENT;
  }
}

uint64_t bmoe_host_tile_count(const uint32_t* counts, uint32_t experts,
                              uint32_t n, uint32_t tile_m, uint32_t tile_n) {
  if (tile_m == 0 || tile_n == 0 || (counts == nullptr && experts != 0)) {
    return std::numeric_limits<uint64_t>::max();
  }
  const uint64_t n_tiles = (static_cast<uint64_t>(n) + tile_n - 1) / tile_n;
  uint64_t total = 0;
  for (uint32_t e = 0; e < experts; ++e) {
    total += ((static_cast<uint64_t>(counts[e]) + tile_m - 1) / tile_m) * n_tiles;
  }
  return total;
}

int bmoe_host_build_tiles(const uint32_t* counts, uint32_t experts, uint32_t n,
                          uint32_t tile_m, uint32_t tile_n, uint32_t order,
                          uint32_t raster, bmoe_tile* tiles_out,
                          uint64_t capacity, uint64_t* count_out) {
  if ((counts == nullptr && experts != 0) || order > 1 || raster > 1 ||
      (tiles_out == nullptr && capacity != 0)) {
    return BMOE_INVALID_ARGUMENT;
  }
  try {
    const bm::GemmShape shape = make_shape(n, tile_m, tile_n);
    const std::vector<uint32_t> tokens = to_vector(counts, experts);
    std::vector<bm::ExpertTile> tiles =
        order == BMOE_ORDER_EXPERT
            ? bm::build_expert_tiles(tokens, shape)
            : bm::order_by_descending_expert_tiles(tokens, shape);
    if (raster == BMOE_RASTER_M_FASTEST) {
      // Same expert visiting order, each expert's grid re-walked column-major.
      std::vector<bm::ExpertTile> rewalked;
      rewalked.reserve(tiles.size());
      std::size_t i = 0;
      while (i < tiles.size()) {
        const uint32_t e = tiles[i].expert_id;
        append_m_fastest(rewalked, e, tokens[e], shape);
        while (i < tiles.size() && tiles[i].expert_id == e) ++i;
      }
      tiles.swap(rewalked);
    }
    if (count_out != nullptr) *count_out = tiles.size();
    const uint64_t n_copy = std::min<uint64_t>(capacity, tiles.size());
    static_assert(sizeof(bmoe_tile) == sizeof(bm::ExpertTile), "record size");
    if (n_copy != 0) {
      std::memcpy(tiles_out, tiles.data(), n_copy * sizeof(bmoe_tile));
    }
    return BMOE_OK;
  } catch (const std::exception&) {
    return BMOE_INVALID_ARGUMENT;
  }
}

int bmoe_host_simulate(uint32_t scheduler, const uint32_t* counts,
                       uint32_t experts, uint32_t n, uint32_t tile_m,
                       uint32_t tile_n, uint32_t cta_count,
                       bmoe_tile* tiles_out, uint64_t capacity,
                       uint64_t* cta_offsets_out,
                       bmoe_schedule_metrics* metrics_out) {
  if ((counts == nullptr && experts != 0) || scheduler > BMOE_SCHED_CLC) {
    return BMOE_INVALID_ARGUMENT;
  }
  try {
    const bm::GemmShape shape = make_shape(n, tile_m, tile_n);
    const bm::CtaAssignment a = bm::simulate_scheduler(
        static_cast<bm::SchedulerKind>(scheduler), to_vector(counts, experts),
        shape, cta_count);
    uint64_t cursor = 0;
    for (std::size_t c = 0; c < a.cta_tiles.size(); ++c) {
      if (cta_offsets_out != nullptr) cta_offsets_out[c] = cursor;
      for (const bm::ExpertTile& t : a.cta_tiles[c]) {
        if (tiles_out != nullptr && cursor < capacity) {
          std::memcpy(&tiles_out[cursor], &t, sizeof(bmoe_tile));
        }
        ++cursor;
      }
    }
    if (cta_offsets_out != nullptr) cta_offsets_out[a.cta_tiles.size()] = cursor;
    if (metrics_out != nullptr) {
      const bm::ScheduleMetrics m = bm::compute_schedule_metrics(a, shape);
      metrics_out->total_tiles = m.total_tiles;
      metrics_out->total_valid_elements = m.total_valid_elements;
      metrics_out->total_padded_elements = m.total_padded_elements;
      metrics_out->expert_switches = m.expert_switches;
      metrics_out->min_tiles_per_cta = m.min_tiles_per_cta;
      metrics_out->max_tiles_per_cta = m.max_tiles_per_cta;
      metrics_out->mean_cta_work = m.mean_cta_work;
      metrics_out->max_cta_work = m.max_cta_work;
      metrics_out->cta_work_cv = m.cta_work_cv;
      metrics_out->tail_ratio = m.tail_ratio;
      metrics_out->estimated_utilization = m.estimated_utilization;
      metrics_out->useful_work_ratio = m.useful_work_ratio;
    }
    return BMOE_OK;
  } catch (const std::exception&) {
    return BMOE_INVALID_ARGUMENT;
  }
}

int bmoe_routing_features_compute(const uint32_t* counts, uint32_t experts,
                                  uint32_t n, uint32_t tile_m, uint32_t tile_n,
                                  uint32_t cta_count,
                                  bmoe_routing_features* out) {
  if (out == nullptr || (counts == nullptr && experts != 0)) {
    return BMOE_INVALID_ARGUMENT;
  }
  try {
    const bm::RoutingFeatures f = bm::routing_features(
        to_vector(counts, experts), make_shape(n, tile_m, tile_n), cta_count);
    out->mean_m = f.mean_m;
    out->cv_m = f.cv_m;
    out->max_over_mean_m = f.max_over_mean_m;
    out->inactive_expert_ratio = f.inactive_expert_ratio;
    out->small_m_expert_ratio = f.small_m_expert_ratio;
    out->expert_tile_cv = f.expert_tile_cv;
    out->max_expert_tiles_over_mean = f.max_expert_tiles_over_mean;
    out->active_tiles = f.active_tiles;
    out->tiles_per_cta = f.tiles_per_cta;
    out->useful_work_ratio = f.useful_work_ratio;
    return BMOE_OK;
  } catch (const std::exception&) {
    return BMOE_INVALID_ARGUMENT;
  }
}

int bmoe_select_variant(const bmoe_routing_features* features,
                        const double* thresholds, uint32_t* variant_out) {
  if (features == nullptr || variant_out == nullptr) {
    return BMOE_INVALID_ARGUMENT;
  }
  bm::RoutingFeatures f;
  f.mean_m = features->mean_m;
  f.cv_m = features->cv_m;
  f.max_over_mean_m = features->max_over_mean_m;
  f.inactive_expert_ratio = features->inactive_expert_ratio;
  f.small_m_expert_ratio = features->small_m_expert_ratio;
  f.expert_tile_cv = features->expert_tile_cv;
  f.max_expert_tiles_over_mean = features->max_expert_tiles_over_mean;
  f.active_tiles = features->active_tiles;
  f.tiles_per_cta = features->tiles_per_cta;
  f.useful_work_ratio = features->useful_work_ratio;
  bm::DispatchThresholds t;
  if (thresholds != nullptr) {
    t.nonpersistent_tiles_per_cta = thresholds[0];
    t.static_cv_m = thresholds[1];
    t.dynamic_min_tiles_per_cta = thresholds[2];
    t.chunked_min_tiles_per_cta = thresholds[3];
    t.high_skew_cv_m = thresholds[4];
    t.sparse_expert_ratio = thresholds[5];
  }
  *variant_out = static_cast<uint32_t>(bm::select_launch_variant(f, t));
  return BMOE_OK;
}

int bmoe_select_variant_fitted(const bmoe_routing_features* features, const double* rule,
                               uint32_t* variant_out) {
  if (features == nullptr || variant_out == nullptr) return BMOE_INVALID_ARGUMENT;
  bm::RoutingFeatures f;
  f.mean_m = features->mean_m;
  f.cv_m = features->cv_m;
  f.inactive_expert_ratio = features->inactive_expert_ratio;
  f.active_tiles = features->active_tiles;
  f.tiles_per_cta = features->tiles_per_cta;
  bm::FittedDispatch r;
  if (rule != nullptr) {
    r.nonpersistent_tiles_per_cta = rule[0];
    r.weight_stream_mean_rows = rule[1];
  }
  *variant_out = static_cast<uint32_t>(bm::select_launch_variant_fitted(f, r));
  return BMOE_OK;
}

const char* bmoe_variant_name(uint32_t variant) {
  if (variant > BMOE_VARIANT_CLC) return "unknown";
  return bm::launch_variant_name(static_cast<bm::LaunchVariant>(variant));
}

}  // extern "C"

namespace blackwell_moe {

// The reference declares this in grouped_gemm.cuh:40 but defines it only in
// its optional CUTLASS baseline; here it is always available.
const char* kernel_status_string(KernelStatus status) {
  return bmoe_status_string(static_cast<int>(status));
}

}  // namespace blackwell_moe
