// Host tile-scheduler model. Behaviour follows src/scheduler/scheduler.cpp of
// the reference:
//   policy names                       scheduler.cpp:11-35
//   build_expert_tiles                 scheduler.cpp:37-60
//   round-robin assignment             scheduler.cpp:62-70
//   descending-work expert order       scheduler.cpp:72-103
//   idealised dynamic queue            scheduler.cpp:105-122
//   simulate_scheduler                 scheduler.cpp:124-145
//   compute_schedule_metrics           scheduler.cpp:147-211
// The device worklist builder (csrc/cuda/worklist.cu) is checked byte for byte
// against these functions.
#include "blackwell_moe/scheduler/scheduler.cuh"

#include <algorithm>
#include <cmath>
#include <limits>
#include <numeric>
#include <stdexcept>

namespace blackwell_moe {

namespace {

void require_tile_dims(const GemmShape& shape) {
  if (shape.tile_m == 0 || shape.tile_n == 0) {
    throw std::invalid_argument("tile dimensions must be positive");
  }
}

std::uint32_t ceil_div(std::uint32_t a, std::uint32_t b) {
  return a == 0 ? 0 : (a + b - 1) / b;
}

// Appends the tile grid of one expert: tile_m outer, tile_n inner.
void append_expert(std::vector<ExpertTile>& out, std::uint32_t expert,
                   std::uint32_t tokens, std::uint32_t n_tiles,
                   const GemmShape& shape) {
  const std::uint32_t m_tiles = ceil_div(tokens, shape.tile_m);
  for (std::uint32_t tm = 0; tm < m_tiles; ++tm) {
    const std::uint32_t rows = std::min(shape.tile_m, tokens - tm * shape.tile_m);
    for (std::uint32_t tn = 0; tn < n_tiles; ++tn) {
      const std::uint32_t cols = std::min(shape.tile_n, shape.n - tn * shape.tile_n);
      out.push_back(ExpertTile{expert, tm, tn, rows, cols});
    }
  }
}

}  // namespace

std::string to_string(SchedulerKind scheduler) {
  switch (scheduler) {
    case SchedulerKind::kExpertOrder: return "expert_order";
    case SchedulerKind::kStaticPersistent: return "static_persistent";
    case SchedulerKind::kDynamicQueue: return "dynamic_queue";
    case SchedulerKind::kCompacted: return "compacted";
    case SchedulerKind::kAuto: return "auto";
    case SchedulerKind::kClc: return "clc";
  }
  throw std::invalid_argument("unknown scheduler");
}

SchedulerKind parse_scheduler(const std::string& value) {
  static const struct { const char* name; SchedulerKind kind; } names[] = {
      {"expert_order", SchedulerKind::kExpertOrder},
      {"baseline", SchedulerKind::kExpertOrder},
      {"static", SchedulerKind::kStaticPersistent},
      {"static_persistent", SchedulerKind::kStaticPersistent},
      {"sorted_static", SchedulerKind::kStaticPersistent},
      {"dynamic", SchedulerKind::kDynamicQueue},
      {"dynamic_queue", SchedulerKind::kDynamicQueue},
      {"compacted", SchedulerKind::kCompacted},
      {"auto", SchedulerKind::kAuto},
      {"clc", SchedulerKind::kClc},
      {"clc_assisted", SchedulerKind::kClc},
  };
  for (const auto& row : names) {
    if (value == row.name) return row.kind;
  }
  throw std::invalid_argument("unknown scheduler: " + value);
}

std::vector<ExpertTile> build_expert_tiles(
    const std::vector<std::uint32_t>& tokens_per_expert,
    const GemmShape& shape,
    bool /*compact_inactive*/) {
  require_tile_dims(shape);
  const std::uint32_t n_tiles = (shape.n + shape.tile_n - 1) / shape.tile_n;
  std::vector<ExpertTile> tiles;
  for (std::uint32_t e = 0; e < tokens_per_expert.size(); ++e) {
    append_expert(tiles, e, tokens_per_expert[e], n_tiles, shape);
  }
  return tiles;
}

std::vector<ExpertTile> order_by_descending_expert_tiles(
    const std::vector<std::uint32_t>& tokens_per_expert,
    const GemmShape& shape) {
  require_tile_dims(shape);
  const std::uint32_t experts =
      static_cast<std::uint32_t>(tokens_per_expert.size());
  const std::uint32_t n_tiles = (shape.n + shape.tile_n - 1) / shape.tile_n;

  // Sort key: tiles of the expert, more first; equal keys keep ascending id.
  std::vector<std::uint64_t> tile_count(experts);
  for (std::uint32_t e = 0; e < experts; ++e) {
    tile_count[e] = static_cast<std::uint64_t>(
                        ceil_div(tokens_per_expert[e], shape.tile_m)) * n_tiles;
  }
  std::vector<std::uint32_t> visit(experts);
  std::iota(visit.begin(), visit.end(), 0u);
  std::stable_sort(visit.begin(), visit.end(),
                   [&tile_count](std::uint32_t a, std::uint32_t b) {
                     return tile_count[a] > tile_count[b];
                   });

  std::vector<ExpertTile> ordered;
  for (std::uint32_t e : visit) {
    append_expert(ordered, e, tokens_per_expert[e], n_tiles, shape);
  }
  return ordered;
}

CtaAssignment assign_expert_order(
    const std::vector<ExpertTile>& tiles, std::uint32_t cta_count) {
  if (cta_count == 0) throw std::invalid_argument("cta_count must be positive");
  CtaAssignment out;
  out.cta_tiles.resize(cta_count);
  std::uint32_t cta = 0;
  for (const ExpertTile& tile : tiles) {
    out.cta_tiles[cta].push_back(tile);
    if (++cta == cta_count) cta = 0;
  }
  return out;
}

CtaAssignment assign_static_persistent(
    const std::vector<std::uint32_t>& tokens_per_expert,
    const GemmShape& shape,
    std::uint32_t cta_count) {
  return assign_expert_order(
      order_by_descending_expert_tiles(tokens_per_expert, shape), cta_count);
}

CtaAssignment assign_dynamic_queue(
    const std::vector<ExpertTile>& tiles, std::uint32_t cta_count) {
  if (cta_count == 0) throw std::invalid_argument("cta_count must be positive");
  CtaAssignment out;
  out.cta_tiles.resize(cta_count);
  std::vector<std::uint64_t> free_at(cta_count, 0);
  for (const ExpertTile& tile : tiles) {
    // Earliest-free CTA; the lowest index wins a tie.
    std::uint32_t best = 0;
    for (std::uint32_t c = 1; c < cta_count; ++c) {
      if (free_at[c] < free_at[best]) best = c;
    }
    out.cta_tiles[best].push_back(tile);
    free_at[best] += std::max<std::uint64_t>(1, valid_output_elements(tile));
  }
  return out;
}

CtaAssignment simulate_scheduler(
    SchedulerKind scheduler,
    const std::vector<std::uint32_t>& tokens_per_expert,
    const GemmShape& shape,
    std::uint32_t cta_count) {
  switch (scheduler) {
    case SchedulerKind::kStaticPersistent:
      return assign_static_persistent(tokens_per_expert, shape, cta_count);
    case SchedulerKind::kDynamicQueue:
    case SchedulerKind::kClc:
      // CLC hands pending tiles to whichever CTA asks first, which the
      // idealised queue models as well; the reference has no CLC entry.
      return assign_dynamic_queue(build_expert_tiles(tokens_per_expert, shape),
                                  cta_count);
    case SchedulerKind::kExpertOrder:
    case SchedulerKind::kCompacted:
    case SchedulerKind::kAuto:
      return assign_expert_order(build_expert_tiles(tokens_per_expert, shape),
                                 cta_count);
  }
  throw std::invalid_argument("unknown scheduler");
}

ScheduleMetrics compute_schedule_metrics(
    const CtaAssignment& assignment, const GemmShape& shape) {
  require_tile_dims(shape);
  ScheduleMetrics m;
  const std::size_t ctas = assignment.cta_tiles.size();
  if (ctas == 0) return m;

  std::vector<double> work(ctas);
  m.min_tiles_per_cta = std::numeric_limits<std::uint64_t>::max();
  for (std::size_t c = 0; c < ctas; ++c) {
    const std::vector<ExpertTile>& list = assignment.cta_tiles[c];
    const std::uint64_t count = list.size();
    m.total_tiles += count;
    m.min_tiles_per_cta = std::min(m.min_tiles_per_cta, count);
    m.max_tiles_per_cta = std::max(m.max_tiles_per_cta, count);
    std::uint64_t valid = 0;
    for (std::size_t i = 0; i < list.size(); ++i) {
      valid += valid_output_elements(list[i]);
      if (i != 0 && list[i].expert_id != list[i - 1].expert_id) {
        ++m.expert_switches;
      }
    }
    m.total_valid_elements += valid;
    work[c] = static_cast<double>(valid);
  }
  m.total_padded_elements =
      m.total_tiles * (static_cast<std::uint64_t>(shape.tile_m) * shape.tile_n);

  double sum = 0.0;
  double peak = work[0];
  for (double w : work) {
    sum += w;
    peak = std::max(peak, w);
  }
  m.mean_cta_work = sum / static_cast<double>(ctas);
  m.max_cta_work = peak;
  if (m.mean_cta_work > 0.0) {
    double ss = 0.0;
    for (double w : work) {
      const double d = w - m.mean_cta_work;
      ss += d * d;
    }
    m.cta_work_cv = std::sqrt(ss / static_cast<double>(ctas)) / m.mean_cta_work;
    m.tail_ratio = m.max_cta_work / m.mean_cta_work;
  }
  if (m.max_cta_work > 0.0) {
    m.estimated_utilization =
        static_cast<double>(m.total_valid_elements) /
        (static_cast<double>(ctas) * m.max_cta_work);
  }
  if (m.total_padded_elements > 0) {
    m.useful_work_ratio = static_cast<double>(m.total_valid_elements) /
                          static_cast<double>(m.total_padded_elements);
  }
  return m;
}

}  // namespace blackwell_moe
