// Dense-plan entry points of the reference, served by the grouped engine with a
// single expert (E = 1, tokens = m):
//   Sm100DenseGemmPlan      src/kernels/sm100_dense_gemm.cu:157-268
//   Sm100TwoSmGemmPlan      src/kernels/sm100_2sm_gemm.cu:150-265
//   launch_direct_cute_gemm src/kernels/direct_cute_gemm.cu:379-414
// Argument checks and status codes follow those functions.
#include <utility>

#include "blackwell_moe/kernels/direct_cute_gemm.cuh"
#include "blackwell_moe/kernels/sm100_2sm_gemm.cuh"
#include "blackwell_moe/kernels/sm100_dense_gemm.cuh"
#include "bmoe_b200.h"

namespace blackwell_moe {

namespace {

// One-expert grouped plan plus the host arrays its arguments point to.
struct DensePlanState {
  bmoe_plan* handle = nullptr;
  const void* a[1] = {nullptr};
  const void* b[1] = {nullptr};
  void* d[1] = {nullptr};
  uint32_t rows[1] = {0};
  Sm100DenseGemmPlanStats stats;
  bool ready = false;

  ~DensePlanState() { bmoe_plan_destroy(handle); }

  KernelStatus initialize(const Sm100DenseGemmArguments& args, uint32_t cta_group,
                          bool output_f32) {
    ready = false;
    stats = Sm100DenseGemmPlanStats{};
    if (args.a == nullptr || args.b == nullptr || args.d == nullptr || args.m == 0 ||
        args.n == 0 || args.k == 0 || args.n % 8 != 0 || args.k % 8 != 0) {
      return KernelStatus::kInvalidArgument;
    }
    if (handle == nullptr) handle = bmoe_plan_create();
    if (handle == nullptr) return KernelStatus::kCudaError;
    a[0] = args.a;
    b[0] = args.b;
    d[0] = args.d;
    rows[0] = args.m;
    bmoe_gemm_args c{};
    c.a = a;
    c.b = b;
    c.d = d;
    c.tokens_per_expert = rows;
    c.experts = 1;
    c.n = args.n;
    c.k = args.k;
    c.scheduler = BMOE_SCHED_CLC;  // the reference collectives use the CLC tile scheduler
    c.cta_group = cta_group;
    // Pairs compute 256 x 256 tiles; the single-CTA plan lets the engine narrow the
    // tile (256 / 128 / 64 columns) until every SM has one, which is what a small-M
    // problem needs to stream its weights at full memory bandwidth.
    c.tile_n = cta_group == 2 ? 256u : 0u;
    c.raster_along_m = -1;
    c.output_f32 = output_f32 ? 1u : 0u;
    c.stream = args.stream;
    const int rc = bmoe_plan_initialize(handle, &c);
    if (rc != BMOE_OK) return static_cast<KernelStatus>(rc);
    bmoe_plan_stats s{};
    bmoe_plan_stats_get(handle, &s);
    stats.workspace_bytes = static_cast<std::size_t>(s.workspace_bytes);
    stats.persistent_ctas = s.threadblock_count;
    stats.tile_m = s.tile_m;
    stats.tile_n = s.tile_n;
    stats.tile_k = 64;
    stats.sm_count = s.sm_count;
    ready = true;
    return KernelStatus::kSuccess;
  }

  KernelStatus run(void* stream) {
    if (!ready) return KernelStatus::kInvalidArgument;
    return static_cast<KernelStatus>(bmoe_plan_run(handle, stream));
  }

  // Waits for the last launch and reports a device-side time-out, if any.
  KernelStatus finish() {
    if (!ready) return KernelStatus::kInvalidArgument;
    return static_cast<KernelStatus>(bmoe_plan_poll(handle, nullptr));
  }
};

}  // namespace

// ------------------------------------------------------------ 1-CTA plan --
struct Sm100DenseGemmPlan::Impl : DensePlanState {};

Sm100DenseGemmPlan::Sm100DenseGemmPlan() : impl_(new Impl) {}
Sm100DenseGemmPlan::~Sm100DenseGemmPlan() { delete impl_; }
Sm100DenseGemmPlan::Sm100DenseGemmPlan(Sm100DenseGemmPlan&& other) noexcept
    : impl_(std::exchange(other.impl_, nullptr)) {}
Sm100DenseGemmPlan& Sm100DenseGemmPlan::operator=(Sm100DenseGemmPlan&& other) noexcept {
  if (this != &other) {
    delete impl_;
    impl_ = std::exchange(other.impl_, nullptr);
  }
  return *this;
}

KernelStatus Sm100DenseGemmPlan::initialize(const Sm100DenseGemmArguments& args) {
  if (impl_ == nullptr) impl_ = new Impl;
  return impl_->initialize(args, 1, false);
}

KernelStatus Sm100DenseGemmPlan::run(void* stream) {
  return impl_ == nullptr ? KernelStatus::kInvalidArgument : impl_->run(stream);
}

Sm100DenseGemmPlanStats Sm100DenseGemmPlan::stats() const {
  return impl_ == nullptr ? Sm100DenseGemmPlanStats{} : impl_->stats;
}

KernelStatus launch_sm100_dense_gemm(const Sm100DenseGemmArguments& args) {
  // The plan owns the worklist and descriptors the kernel reads: wait for the
  // launch before it goes out of scope, and report a device-side time-out.
  DensePlanState plan;
  KernelStatus status = plan.initialize(args, 1, false);
  if (status == KernelStatus::kSuccess) status = plan.run(args.stream);
  return status == KernelStatus::kSuccess ? plan.finish() : status;
}

const char* sm100_dense_kernel_name() {
  return "sm100_1cta_persistent_clc_tma_tcgen05_bf16_128x256x64";
}

// ------------------------------------------------------------ CTA-pair plan --
struct Sm100TwoSmGemmPlan::Impl : DensePlanState {};

Sm100TwoSmGemmPlan::Sm100TwoSmGemmPlan() : impl_(new Impl) {}
Sm100TwoSmGemmPlan::~Sm100TwoSmGemmPlan() { delete impl_; }
Sm100TwoSmGemmPlan::Sm100TwoSmGemmPlan(Sm100TwoSmGemmPlan&& other) noexcept
    : impl_(std::exchange(other.impl_, nullptr)) {}
Sm100TwoSmGemmPlan& Sm100TwoSmGemmPlan::operator=(Sm100TwoSmGemmPlan&& other) noexcept {
  if (this != &other) {
    delete impl_;
    impl_ = std::exchange(other.impl_, nullptr);
  }
  return *this;
}

KernelStatus Sm100TwoSmGemmPlan::initialize(const Sm100DenseGemmArguments& args) {
  if (impl_ == nullptr) impl_ = new Impl;
  return impl_->initialize(args, 2, false);
}

KernelStatus Sm100TwoSmGemmPlan::run(void* stream) {
  return impl_ == nullptr ? KernelStatus::kInvalidArgument : impl_->run(stream);
}

Sm100DenseGemmPlanStats Sm100TwoSmGemmPlan::stats() const {
  return impl_ == nullptr ? Sm100DenseGemmPlanStats{} : impl_->stats;
}

KernelStatus launch_sm100_2sm_gemm(const Sm100DenseGemmArguments& args) {
  DensePlanState plan;
  KernelStatus status = plan.initialize(args, 2, false);
  if (status == KernelStatus::kSuccess) status = plan.run(args.stream);
  return status == KernelStatus::kSuccess ? plan.finish() : status;
}

const char* sm100_2sm_kernel_name() {
  return "sm100_cta_pair_persistent_clc_tma_tcgen05_bf16_256x256x64";
}

// ------------------------------------------------------- FP32-output one-shot --
KernelStatus launch_direct_cute_gemm(const DirectCuteGemmArguments& args,
                                     DirectCuteGemmStats* stats) {
  if (args.a == nullptr || args.b == nullptr || args.d == nullptr || args.m == 0 ||
      args.n == 0 || args.k == 0 || args.m % 128 != 0 || args.n % 256 != 0 ||
      args.k % 64 != 0 || args.m > 0x7fffffffu || args.n > 0x7fffffffu ||
      args.k > 0x7fffffffu) {
    return KernelStatus::kInvalidArgument;
  }
  Sm100DenseGemmArguments dense;
  dense.a = args.a;
  dense.b = args.b;
  dense.d = args.d;
  dense.m = args.m;
  dense.n = args.n;
  dense.k = args.k;
  dense.stream = args.stream;
  DensePlanState plan;
  KernelStatus status = plan.initialize(dense, 1, true);
  if (status != KernelStatus::kSuccess) return status;
  status = plan.run(args.stream);
  if (status != KernelStatus::kSuccess) return status;
  if (stats != nullptr) {
    stats->grid_m = args.m / 128;
    stats->grid_n = args.n / 256;
    stats->tile_m = 128;
    stats->tile_n = 256;
    stats->tile_k = 64;
    bmoe_plan_stats s{};
    bmoe_plan_stats_get(plan.handle, &s);
    stats->dynamic_smem_bytes = s.dynamic_smem_bytes;
  }
  return static_cast<KernelStatus>(bmoe_plan_poll(plan.handle, nullptr));
}

const char* direct_cute_kernel_name() {
  return "sm100_tma_tcgen05_tmem_bf16_f32_128x256x64";
}

}  // namespace blackwell_moe
