// C++ classes of include/blackwell_moe/kernels/grouped_gemm.cuh and
// scheduler_probe.cuh, implemented as thin wrappers over the C interface
// (bmoe_b200.h). Semantics follow the reference implementations:
//   Bf16GroupedGemmPlan / launch_grouped_gemm_baseline
//       baselines/cutlass/cutlass_baseline.cu:179-387
//   launch_scheduler_probe / device_scheduler_name
//       src/kernels/scheduler_probe.cu:105-141
#include <utility>

#include "blackwell_moe/kernels/grouped_gemm.cuh"
#include "blackwell_moe/scheduler/scheduler_probe.cuh"
#include "bmoe_b200.h"

namespace blackwell_moe {

namespace {

bmoe_gemm_args to_c_args(const GroupedGemmArguments& args) {
  bmoe_gemm_args c{};
  c.a = args.a;
  c.b = args.b;
  c.d = args.d;
  c.tokens_per_expert = args.tokens_per_expert;
  c.experts = args.experts;
  c.n = args.n;
  c.k = args.k;
  c.data_type = static_cast<uint32_t>(args.data_type);
  c.scheduler = static_cast<uint32_t>(args.scheduler);
  c.claim_size = args.claim_size;
  c.hybrid_tail_tiles = args.hybrid_tail_tiles;
  c.cta_count = args.cta_count;
  c.tile_n = args.tile_n;
  c.cta_group = args.cta_group;
  c.raster_along_m = args.raster_along_m;
  c.output_f32 = 0;
  c.stream = args.stream;
  return c;
}

}  // namespace

struct Bf16GroupedGemmPlan::Impl {
  bmoe_plan* handle = nullptr;
  ~Impl() { bmoe_plan_destroy(handle); }
};

Bf16GroupedGemmPlan::Bf16GroupedGemmPlan() : impl_(new Impl) {}

Bf16GroupedGemmPlan::~Bf16GroupedGemmPlan() { delete impl_; }

Bf16GroupedGemmPlan::Bf16GroupedGemmPlan(Bf16GroupedGemmPlan&& other) noexcept
    : impl_(std::exchange(other.impl_, nullptr)) {}

Bf16GroupedGemmPlan& Bf16GroupedGemmPlan::operator=(
    Bf16GroupedGemmPlan&& other) noexcept {
  if (this != &other) {
    delete impl_;
    impl_ = std::exchange(other.impl_, nullptr);
  }
  return *this;
}

KernelStatus Bf16GroupedGemmPlan::initialize(const GroupedGemmArguments& args) {
  // The BF16 plan takes BF16 only, as the reference's does (after its argument checks:
  // cutlass_baseline.cu:206-213). The engine checks arguments first, then the type.
  if (args.data_type != DataType::kBf16) {
    GroupedGemmArguments probe = args;
    probe.data_type = static_cast<DataType>(0x7fffffff);
    return initialize_typed(probe);
  }
  return initialize_typed(args);
}

KernelStatus Fp8E4m3GroupedGemmPlan::initialize(const GroupedGemmArguments& args) {
  if (args.data_type != DataType::kFp8E4M3) {
    GroupedGemmArguments probe = args;
    probe.data_type = static_cast<DataType>(0x7fffffff);
    return plan_.initialize_typed(probe);
  }
  return plan_.initialize_typed(args);
}

KernelStatus Bf16GroupedGemmPlan::initialize_typed(const GroupedGemmArguments& args) {
  if (impl_ == nullptr) impl_ = new Impl;
  if (impl_->handle == nullptr) impl_->handle = bmoe_plan_create();
  if (impl_->handle == nullptr) return KernelStatus::kCudaError;
  const bmoe_gemm_args c = to_c_args(args);
  return static_cast<KernelStatus>(bmoe_plan_initialize(impl_->handle, &c));
}

KernelStatus Bf16GroupedGemmPlan::run(void* stream) {
  if (impl_ == nullptr || impl_->handle == nullptr) {
    return KernelStatus::kInvalidArgument;
  }
  return static_cast<KernelStatus>(bmoe_plan_run(impl_->handle, stream));
}

GroupedGemmPlanStats Bf16GroupedGemmPlan::stats() const {
  GroupedGemmPlanStats out;
  if (impl_ == nullptr || impl_->handle == nullptr) return out;
  bmoe_plan_stats s{};
  bmoe_plan_stats_get(impl_->handle, &s);
  out.active_experts = s.active_experts;
  out.threadblock_count = s.threadblock_count;
  out.workspace_bytes = static_cast<std::size_t>(s.workspace_bytes);
  out.total_tiles = s.total_tiles;
  out.tile_m = s.tile_m;
  out.tile_n = s.tile_n;
  out.resolved_scheduler = static_cast<SchedulerKind>(s.resolved_scheduler);
  out.claim_size = s.claim_size;
  out.hybrid_tail_tiles = s.hybrid_tail_tiles;
  return out;
}

KernelStatus Bf16GroupedGemmPlan::poll() {
  if (impl_ == nullptr || impl_->handle == nullptr) {
    return KernelStatus::kInvalidArgument;
  }
  return static_cast<KernelStatus>(bmoe_plan_poll(impl_->handle, nullptr));
}

KernelStatus Bf16GroupedGemmPlan::set_exchange_gate(const std::uint32_t* flags,
                                                    std::uint32_t epoch, std::uint32_t ranks,
                                                    std::uint32_t self,
                                                    const std::uint8_t* group_of_expert) {
  if (impl_ == nullptr || impl_->handle == nullptr) return KernelStatus::kInvalidArgument;
  return static_cast<KernelStatus>(
      bmoe_plan_set_gate(impl_->handle, flags, epoch, ranks, self, group_of_expert));
}

KernelStatus Bf16GroupedGemmPlan::set_result_push(const void* origin,
                                                  const std::uint32_t* expert_first_row,
                                                  void* const* y_bases, std::uint32_t ranks,
                                                  std::uint64_t y_rows_cap) {
  if (impl_ == nullptr || impl_->handle == nullptr) return KernelStatus::kInvalidArgument;
  return static_cast<KernelStatus>(
      bmoe_plan_set_push(impl_->handle, origin, expert_first_row, y_bases, ranks, y_rows_cap));
}

void* Bf16GroupedGemmPlan::native_handle() const {
  return impl_ == nullptr ? nullptr : impl_->handle;
}

KernelStatus launch_grouped_gemm_baseline(const GroupedGemmArguments& args) {
  bmoe_gemm_args c = to_c_args(args);
  if (args.data_type != DataType::kBf16) c.data_type = 0x7fffffffu;  // BF16 only, as above
  return static_cast<KernelStatus>(bmoe_grouped_gemm(&c));
}

KernelStatus launch_scheduler_probe(DeviceSchedulerKind scheduler,
                                    const SchedulerProbeArguments& args) {
  static_assert(sizeof(ExpertTile) == sizeof(bmoe_tile), "tile record layout");
  bmoe_probe_args c{};
  c.tiles = reinterpret_cast<const bmoe_tile*>(args.tiles);
  c.tile_count = args.tile_count;
  c.cta_count = args.cta_count;
  c.claim_size = args.claim_size;
  c.work_scale = args.work_scale;
  c.next_tile = args.next_tile;
  c.tile_visits = args.tile_visits;
  c.tile_checksums = args.tile_checksums;
  c.cta_tile_counts = args.cta_tile_counts;
  c.cta_valid_elements = args.cta_valid_elements;
  c.stream = args.stream;
  return static_cast<KernelStatus>(
      bmoe_probe_launch(static_cast<uint32_t>(scheduler), &c));
}

const char* device_scheduler_name(DeviceSchedulerKind scheduler) {
  return bmoe_probe_scheduler_name(static_cast<uint32_t>(scheduler));
}

}  // namespace blackwell_moe
