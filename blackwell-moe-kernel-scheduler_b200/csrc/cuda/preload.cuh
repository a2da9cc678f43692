// Forces the CUDA module of every kernel of the library to load now (kernels load
// lazily on their first launch otherwise, which can take tens of milliseconds and
// differ between the ranks of a multi-GPU step that waits on flags).
#pragma once

#include <cuda_runtime.h>

namespace bmoe {

cudaError_t preload_gemm_kernels();
cudaError_t preload_worklist_kernels();
cudaError_t preload_permute_kernels();
cudaError_t preload_exchange_kernels();
cudaError_t preload_probe_kernels();

template <typename Kernel>
cudaError_t preload_one(Kernel kernel) {
  cudaFuncAttributes attributes;
  return cudaFuncGetAttributes(&attributes, kernel);
}

}  // namespace bmoe
