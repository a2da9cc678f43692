// Dense BF16 GEMM plan on CTA pairs: two CTAs of a cluster compute one
// 256 x 256 tile with tcgen05 cta_group::2, each loading its own operand halves
// with plain TMA (no multicast).
//
// Source-compatible with the reference interface
// include/blackwell_moe/kernels/sm100_2sm_gemm.cuh:13-33 (a CUTLASS 2-SM
// collective with TMA multicast there).
#pragma once

#include "blackwell_moe/kernels/sm100_dense_gemm.cuh"

namespace blackwell_moe {

class Sm100TwoSmGemmPlan {
 public:
  Sm100TwoSmGemmPlan();
  ~Sm100TwoSmGemmPlan();

  Sm100TwoSmGemmPlan(const Sm100TwoSmGemmPlan&) = delete;
  Sm100TwoSmGemmPlan& operator=(const Sm100TwoSmGemmPlan&) = delete;
  Sm100TwoSmGemmPlan(Sm100TwoSmGemmPlan&& other) noexcept;
  Sm100TwoSmGemmPlan& operator=(Sm100TwoSmGemmPlan&& other) noexcept;

  KernelStatus initialize(const Sm100DenseGemmArguments& args);
  KernelStatus run(void* stream = nullptr);
  Sm100DenseGemmPlanStats stats() const;

 private:
  struct Impl;
  Impl* impl_ = nullptr;
};

KernelStatus launch_sm100_2sm_gemm(const Sm100DenseGemmArguments& args);
const char* sm100_2sm_kernel_name();

}  // namespace blackwell_moe
