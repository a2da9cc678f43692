// kernel_status_string for programs built from the REFERENCE's own native sm_100a
// kernel sources. The reference declares the function in
// include/blackwell_moe/kernels/grouped_gemm.cuh:40 but defines it only inside its
// optional CUTLASS SM80 baseline (baselines/cutlass/cutlass_baseline.cu:165-176), so
// its native dense benchmark and test do not link without that baseline. This file
// supplies the missing definition for those comparison programs. TEST / BENCHMARK
// INFRASTRUCTURE ONLY: compiled against the reference's headers, never linked into
// the engine library.
#include "blackwell_moe/kernels/grouped_gemm.cuh"

namespace blackwell_moe {

const char* kernel_status_string(KernelStatus status) {
  static const char* const names[] = {
      "success",           "invalid argument", "unsupported data type",
      "unsupported scheduler", "unsupported device", "CUDA error", "CUTLASS error"};
  const int index = static_cast<int>(status);
  return index >= 0 && index < 7 ? names[index] : "unknown status";
}

}  // namespace blackwell_moe
