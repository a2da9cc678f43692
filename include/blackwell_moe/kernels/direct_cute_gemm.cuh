// One-shot dense GEMM with FP32 output:
//   D_f32[m, n] = A_bf16[m, k] * B_bf16[n, k]^T     (the unrounded accumulators)
// Complete 128 x 256 x 64 tiles only, as in the reference bring-up contract
// include/blackwell_moe/kernels/direct_cute_gemm.cuh:16-39; served by the
// grouped engine's FP32 epilogue.
#pragma once

#include <cstddef>
#include <cstdint>

#include "blackwell_moe/kernels/grouped_gemm.cuh"

namespace blackwell_moe {

struct DirectCuteGemmArguments {
  const void* a = nullptr;  // row-major BF16 [m, k]
  const void* b = nullptr;  // row-major BF16 [n, k]
  void* d = nullptr;        // row-major FP32 [m, n]
  std::uint32_t m = 0;      // multiple of 128
  std::uint32_t n = 0;      // multiple of 256
  std::uint32_t k = 0;      // multiple of 64
  void* stream = nullptr;
};

struct DirectCuteGemmStats {
  std::uint32_t grid_m = 0;
  std::uint32_t grid_n = 0;
  std::uint32_t tile_m = 128;
  std::uint32_t tile_n = 256;
  std::uint32_t tile_k = 64;
  std::size_t dynamic_smem_bytes = 0;
};

// Synchronous with respect to plan storage: returns after the kernel finished.
KernelStatus launch_direct_cute_gemm(const DirectCuteGemmArguments& args,
                                     DirectCuteGemmStats* stats = nullptr);

const char* direct_cute_kernel_name();

}  // namespace blackwell_moe
