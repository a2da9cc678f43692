// Dense BF16 GEMM plan, D[m, n] = A[m, k] * B[n, k]^T (FP32 accumulate, BF16
// out), served by the grouped engine as a single-expert problem: one CTA per
// 128 x 256 output tile walk, tcgen05 + TMEM + TMA, persistent.
//
// Source-compatible with the reference interface
// include/blackwell_moe/kernels/sm100_dense_gemm.cuh:15-59 (a CUTLASS 1-SM
// collective there).
#pragma once

#include <cstddef>
#include <cstdint>

#include "blackwell_moe/kernels/grouped_gemm.cuh"

namespace blackwell_moe {

// a: row-major [m, k]; b: row-major [n, k]; d: row-major [m, n]; device
// pointers, 16-byte aligned; n and k multiples of 8.
struct Sm100DenseGemmArguments {
  const void* a = nullptr;
  const void* b = nullptr;
  void* d = nullptr;
  std::uint32_t m = 0;
  std::uint32_t n = 0;
  std::uint32_t k = 0;
  void* stream = nullptr;
};

struct Sm100DenseGemmPlanStats {
  std::size_t workspace_bytes = 0;
  std::uint32_t sm_count = 0;
  std::uint32_t persistent_ctas = 0;
  std::uint32_t tile_m = 128;
  std::uint32_t tile_n = 128;
  std::uint32_t tile_k = 64;
};

class Sm100DenseGemmPlan {
 public:
  Sm100DenseGemmPlan();
  ~Sm100DenseGemmPlan();

  Sm100DenseGemmPlan(const Sm100DenseGemmPlan&) = delete;
  Sm100DenseGemmPlan& operator=(const Sm100DenseGemmPlan&) = delete;
  Sm100DenseGemmPlan(Sm100DenseGemmPlan&& other) noexcept;
  Sm100DenseGemmPlan& operator=(Sm100DenseGemmPlan&& other) noexcept;

  KernelStatus initialize(const Sm100DenseGemmArguments& args);
  KernelStatus run(void* stream = nullptr);
  Sm100DenseGemmPlanStats stats() const;

 private:
  struct Impl;
  Impl* impl_ = nullptr;
};

KernelStatus launch_sm100_dense_gemm(const Sm100DenseGemmArguments& args);
const char* sm100_dense_kernel_name();

}  // namespace blackwell_moe
