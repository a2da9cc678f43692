// Scheduler probe: runs the static round-robin and atomic-queue persistent
// loops over integer stand-in work so that exact-once coverage and the
// realised per-CTA balance can be checked without any GEMM math.
//
// Source-compatible with the reference interface
// include/blackwell_moe/scheduler/scheduler_probe.cuh:10-36.
#pragma once

#include <cstdint>

#include "blackwell_moe/kernels/grouped_gemm.cuh"
#include "blackwell_moe/work_tile.cuh"

namespace blackwell_moe {

enum class DeviceSchedulerKind : std::uint32_t {
  kStaticPersistent = 0,
  kDynamicQueue = 1,
};

// All pointers are device pointers. The caller zeroes next_tile, tile_visits
// and the per-CTA counters before a launch.
struct SchedulerProbeArguments {
  const ExpertTile* tiles = nullptr;
  std::uint32_t tile_count = 0;
  std::uint32_t cta_count = 0;
  std::uint32_t claim_size = 1;
  std::uint32_t work_scale = 1;
  std::uint32_t* next_tile = nullptr;           // required for kDynamicQueue
  std::uint32_t* tile_visits = nullptr;         // [tile_count], +1 per visit
  std::uint64_t* tile_checksums = nullptr;      // [tile_count]
  std::uint32_t* cta_tile_counts = nullptr;     // [cta_count]
  std::uint64_t* cta_valid_elements = nullptr;  // [cta_count]
  void* stream = nullptr;
};

KernelStatus launch_scheduler_probe(
    DeviceSchedulerKind scheduler,
    const SchedulerProbeArguments& args);

const char* device_scheduler_name(DeviceSchedulerKind scheduler);

}  // namespace blackwell_moe
