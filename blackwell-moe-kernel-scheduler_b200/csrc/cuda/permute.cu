// Row gather: dst[i, :] = src[index[i], :] for BF16 token rows. Used either side
// of the grouped GEMM: token rows -> send order (one copy per routed expert),
// received rows -> expert-major packed A, and the inverse on the way back.
// The reference treats this permutation as an input of the engine
// (agent/search_space.yaml:13); it is the data format the expert-parallel
// dispatch / combine needs. HBM-bound: 2 * row_bytes per row.
#include <cuda_runtime.h>

#include <cstdint>

#include "bmoe_b200.h"

namespace bmoe {
namespace {

constexpr uint32_t kGatherThreads = 256;

// One warp per row, 16 bytes per lane and step; rows are multiples of 16 bytes.
__global__ void __launch_bounds__(kGatherThreads)
gather_rows_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst,
                   const int64_t* __restrict__ index, uint64_t rows,
                   uint32_t vec_per_row, uint64_t src_rows) {
  const uint32_t lane = threadIdx.x & 31;
  const uint64_t warps = static_cast<uint64_t>(gridDim.x) * (kGatherThreads / 32);
  for (uint64_t r = static_cast<uint64_t>(blockIdx.x) * (kGatherThreads / 32) +
                    (threadIdx.x >> 5);
       r < rows; r += warps) {
    const int64_t from = index[r];
    if (from < 0 || static_cast<uint64_t>(from) >= src_rows) continue;  // skip bad index
    const uint4* s = src + static_cast<uint64_t>(from) * vec_per_row;
    uint4* d = dst + r * vec_per_row;
    for (uint32_t v = lane; v < vec_per_row; v += 32) d[v] = __ldg(s + v);
  }
}

}  // namespace
}  // namespace bmoe

extern "C" int bmoe_gather_rows(const void* src_dev, void* dst_dev,
                                const int64_t* index_dev, uint64_t rows,
                                uint64_t src_rows, uint32_t row_bytes, void* stream) {
  if (rows == 0) return BMOE_OK;
  if (src_dev == nullptr || dst_dev == nullptr || index_dev == nullptr ||
      row_bytes == 0 || row_bytes % 16 != 0 ||
      (reinterpret_cast<uintptr_t>(src_dev) & 15u) != 0 ||
      (reinterpret_cast<uintptr_t>(dst_dev) & 15u) != 0) {
    return BMOE_INVALID_ARGUMENT;
  }
  const uint64_t want = (rows + 7) / 8;                 // 8 warps (rows) per CTA
  const uint32_t grid = static_cast<uint32_t>(want < 148ull * 16 ? want : 148ull * 16);
  bmoe::gather_rows_kernel<<<grid, bmoe::kGatherThreads, 0,
                             static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(src_dev), static_cast<uint4*>(dst_dev), index_dev, rows,
      row_bytes / 16, src_rows);
  return cudaPeekAtLastError() == cudaSuccess ? BMOE_OK : BMOE_CUDA_ERROR;
}
