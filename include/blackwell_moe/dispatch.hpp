// Launch-level routing features, the threshold ("auto") dispatch rule and the
// claim-order models of the in-kernel tile schedulers.
//
// C++ statement of the reference's Python host logic:
//   RoutingFeatures / DispatchThresholds / routing_features / select_kernel
//     python/blackwell_moe_tirx/dispatch.py:16-114
//   static_cta_assignments / chunked_claims / hybrid_claims
//     python/blackwell_moe_tirx/config.py:222-267
// Threshold values and the order of the rules are the reference's.
#pragma once

#include <cstdint>
#include <vector>

#include "blackwell_moe/problem.hpp"
#include "blackwell_moe/scheduler/scheduler.cuh"

namespace blackwell_moe {

struct RoutingFeatures {
  double mean_m = 0.0;
  double cv_m = 0.0;
  double max_over_mean_m = 0.0;
  double inactive_expert_ratio = 0.0;
  // Share of ACTIVE experts with count <= tile_m (differs on purpose from
  // WorkloadMetrics::small_m_expert_ratio; dispatch.py:57-59).
  double small_m_expert_ratio = 0.0;
  double expert_tile_cv = 0.0;
  double max_expert_tiles_over_mean = 0.0;
  std::uint64_t active_tiles = 0;
  double tiles_per_cta = 0.0;
  double useful_work_ratio = 1.0;
};

struct DispatchThresholds {
  double nonpersistent_tiles_per_cta = 1.0;
  double static_cv_m = 0.25;
  double dynamic_min_tiles_per_cta = 2.0;
  double chunked_min_tiles_per_cta = 4.0;
  double high_skew_cv_m = 1.0;
  double sparse_expert_ratio = 0.5;
};

// The engine's own rule for kAuto, fitted on B200 measurements of this engine (the
// reference's rule and bootstrap thresholds above stay available unchanged through
// select_launch_variant / bmoe_select_variant / select_kernel). Fitted on the
// Qwen3-shaped skew sweep (E=128, 131072 rows, N=768, K=2048; uniform and Zipf 0.5 / 1.0 /
// 1.5) and the DeepSeek-shaped decode routing; checked on routings it was not fitted on
// (Mixtral-shaped Zipf 1.0, the four E=64 rows the reference published, the small
// CPU-runnable case), where it stays within 1 % of the best policy's median. What the
// measurements say: launch control (one CTA per tile, work stealing) is the fastest or
// within 0.3 % of it wherever tiles carry real rows; the chunked and hybrid queues never
// paid (5-15 % slower: concurrent tiles then span more weight column blocks); when the
// experts hold only a handful of rows each the launch is a pure weight stream of
// equal-cost tiles and the plain static stride wins by 1-2 % (no claim traffic, and the
// producer may run further ahead of the scheduler).
struct FittedDispatch {
  double nonpersistent_tiles_per_cta = 1.0;   // the reference's value, not contradicted
  // mean rows per ACTIVE expert at or below which the launch counts as a weight stream
  double weight_stream_mean_rows = 32.0;
};

// The launch variants the rule can choose (reference kernel names in
// python/blackwell_moe_tirx/kernels/registry.py:45-106).
enum class LaunchVariant {
  kNonPersistent,   // "v0_nonpersistent": one CTA per tile
  kStaticWs,        // "v1_static_ws":     static grid stride
  kDynamicClaim1,   // "v2_dynamic":       atomic queue, claim 1
  kChunked,         // "v3_chunked":       atomic queue, claim `claim_size`
  kHybrid,          // "v4_hybrid":        coarse chunks + claim-1 tail
  kClc,             // "v5_clc":           never chosen by the reference's rule
};

const char* launch_variant_name(LaunchVariant variant);

// Engine launch configuration for one variant.
struct LaunchConfig {
  LaunchVariant variant = LaunchVariant::kStaticWs;
  SchedulerKind scheduler = SchedulerKind::kStaticPersistent;
  std::uint32_t claim_size = 1;
  std::uint32_t hybrid_tail_tiles = 0;
  bool one_cta_per_tile = false;
};

// Defaults of the reference spec (config.py:31-35).
struct DispatchSpec {
  std::uint32_t cta_count = 148;
  std::uint32_t claim_size = 4;
  std::uint32_t hybrid_main_claim_size = 8;
  std::uint32_t hybrid_tail_tiles = 296;
};

RoutingFeatures routing_features(
    const std::vector<std::uint32_t>& tokens_per_expert,
    const GemmShape& shape,
    std::uint32_t cta_count);

LaunchVariant select_launch_variant(
    const RoutingFeatures& features,
    const DispatchThresholds& thresholds = DispatchThresholds());

// The engine's fitted rule (see FittedDispatch): one CTA per tile when every unit gets
// at most one tile, the static stride for weight-stream routings, launch control
// otherwise.
LaunchVariant select_launch_variant_fitted(
    const RoutingFeatures& features, const FittedDispatch& rule = FittedDispatch());

LaunchConfig resolve_launch_config(
    LaunchVariant variant, const DispatchSpec& spec = DispatchSpec());

// Tile indices each CTA visits under the static grid stride.
std::vector<std::vector<std::uint32_t>> static_cta_assignments(
    std::uint32_t tile_count, std::uint32_t cta_count);
// Contiguous batches handed out by a monotonic atomic queue.
std::vector<std::vector<std::uint32_t>> chunked_claims(
    std::uint32_t tile_count, std::uint32_t claim_size);
// Coarse chunks up to tile_count - min(tile_count, tail_tiles), then singles.
std::vector<std::vector<std::uint32_t>> hybrid_claims(
    std::uint32_t tile_count, std::uint32_t main_claim_size,
    std::uint32_t tail_tiles);

}  // namespace blackwell_moe
