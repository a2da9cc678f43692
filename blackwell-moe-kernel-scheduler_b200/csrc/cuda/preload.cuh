// Forces the CUDA module of every kernel of the library to load now (kernels load
// lazily on their first launch otherwise, which can take tens of milliseconds and
// differ between the ranks of a multi-GPU step that waits on flags).
#pragma once

#include <cuda_runtime.h>

#include <cstdint>

namespace bmoe {

cudaError_t preload_gemm_kernels();
cudaError_t preload_worklist_kernels();
cudaError_t preload_permute_kernels();
cudaError_t preload_exchange_kernels();
cudaError_t preload_probe_kernels();

// SM count of the current device (148 on B200; partitions and other parts differ).
inline uint32_t device_sm_count() {
  int device = 0, sms = 0;
  if (cudaGetDevice(&device) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess ||
      sms <= 0) {
    return 148u;
  }
  return static_cast<uint32_t>(sms);
}

template <typename Kernel>
cudaError_t preload_one(Kernel kernel) {
  cudaFuncAttributes attributes;
  return cudaFuncGetAttributes(&attributes, kernel);
}

}  // namespace bmoe
