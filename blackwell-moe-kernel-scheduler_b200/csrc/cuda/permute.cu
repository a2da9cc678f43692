// Row gather: dst[i, :] = src[index[i], :] for BF16 token rows. Used either side
// of the grouped GEMM: token rows -> send order (one copy per routed expert),
// received rows -> expert-major packed A, and the inverse on the way back.
// The reference treats this permutation as an input of the engine
// (agent/search_space.yaml:13); it is the data format the expert-parallel
// dispatch / combine needs. HBM-bound: 2 * row_bytes per row.
#include <cuda_runtime.h>

#include <cstdint>
#include <cstring>

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

// ------------------------------------------------------------------------
// Row routing over peer memory: one pass moves rows between buffers that may
// live on different GPUs of the node (peer pointers over NVLink),
//   dst_base[dst_rank[i]] + dst_row[i]  <-  src_base[src_rank[i]] + src_row[i].
// With a local source and per-row destination GPUs it is the expert-parallel
// dispatch (token rows pushed straight into the owner's expert-major A); with
// per-row source GPUs and a local destination it is the combine (result rows
// pulled back into assignment order). Plain loads and stores only.
// ------------------------------------------------------------------------
namespace bmoe {
namespace {

constexpr uint32_t kRouteThreads = 256;
constexpr uint32_t kRouteUnroll = 8;  // 16-byte vectors in flight per lane

struct RouteArgs {
  const uint4* const* src_bases;  // [n_src] device array of base pointers
  const int32_t* src_rank;        // [rows] or nullptr (all from src_bases[0])
  const int64_t* src_row;         // [rows] or nullptr (row i)
  uint4* const* dst_bases;        // [n_dst]
  const int32_t* dst_rank;        // [rows] or nullptr
  const int64_t* dst_row;         // [rows] or nullptr (row i)
  uint64_t rows;
  uint32_t vec_per_row;
  uint32_t n_src;
  uint32_t n_dst;
  uint64_t src_rows_cap;          // rows each source buffer holds
  uint64_t dst_rows_cap;
};

__global__ void __launch_bounds__(kRouteThreads) route_rows_kernel(RouteArgs a) {
  const uint32_t lane = threadIdx.x & 31;
  const uint64_t warps = static_cast<uint64_t>(gridDim.x) * (kRouteThreads / 32);
  for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * (kRouteThreads / 32) +
                    (threadIdx.x >> 5);
       i < a.rows; i += warps) {
    const int64_t from_rank = a.src_rank != nullptr ? a.src_rank[i] : 0;
    const int64_t to_rank = a.dst_rank != nullptr ? a.dst_rank[i] : 0;
    const int64_t from_row = a.src_row != nullptr ? a.src_row[i] : static_cast<int64_t>(i);
    const int64_t to_row = a.dst_row != nullptr ? a.dst_row[i] : static_cast<int64_t>(i);
    // A bad index must never become a stray access to another GPU's memory.
    if (from_rank < 0 || from_rank >= a.n_src || to_rank < 0 || to_rank >= a.n_dst ||
        from_row < 0 || static_cast<uint64_t>(from_row) >= a.src_rows_cap || to_row < 0 ||
        static_cast<uint64_t>(to_row) >= a.dst_rows_cap) {
      continue;
    }
    const uint4* s = a.src_bases[from_rank] + static_cast<uint64_t>(from_row) * a.vec_per_row;
    uint4* d = a.dst_bases[to_rank] + static_cast<uint64_t>(to_row) * a.vec_per_row;
    for (uint32_t v0 = 0; v0 < a.vec_per_row; v0 += 32 * kRouteUnroll) {
      uint4 regs[kRouteUnroll];
#pragma unroll
      for (uint32_t u = 0; u < kRouteUnroll; ++u) {
        const uint32_t v = v0 + u * 32 + lane;
        if (v < a.vec_per_row) regs[u] = s[v];
      }
#pragma unroll
      for (uint32_t u = 0; u < kRouteUnroll; ++u) {
        const uint32_t v = v0 + u * 32 + lane;
        if (v < a.vec_per_row) d[v] = regs[u];
      }
    }
  }
}

}  // namespace
}  // namespace bmoe

extern "C" int bmoe_route_rows(const void* const* src_bases_dev, uint32_t n_src,
                               uint64_t src_rows_cap, const int32_t* src_rank_dev,
                               const int64_t* src_row_dev, void* const* dst_bases_dev,
                               uint32_t n_dst, uint64_t dst_rows_cap,
                               const int32_t* dst_rank_dev, const int64_t* dst_row_dev,
                               uint64_t rows, uint32_t row_bytes, uint32_t max_ctas,
                               void* stream) {
  if (rows == 0) return BMOE_OK;
  if (src_bases_dev == nullptr || dst_bases_dev == nullptr || n_src == 0 || n_dst == 0 ||
      row_bytes == 0 || row_bytes % 16 != 0) {
    return BMOE_INVALID_ARGUMENT;
  }
  bmoe::RouteArgs a;
  a.src_bases = reinterpret_cast<const uint4* const*>(src_bases_dev);
  a.src_rank = src_rank_dev;
  a.src_row = src_row_dev;
  a.dst_bases = reinterpret_cast<uint4* const*>(dst_bases_dev);
  a.dst_rank = dst_rank_dev;
  a.dst_row = dst_row_dev;
  a.rows = rows;
  a.vec_per_row = row_bytes / 16;
  a.n_src = n_src;
  a.n_dst = n_dst;
  a.src_rows_cap = src_rows_cap;
  a.dst_rows_cap = dst_rows_cap;
  const uint64_t want = (rows + 7) / 8;
  uint64_t cap = max_ctas != 0 ? max_ctas : 148ull * 8;
  const uint32_t grid = static_cast<uint32_t>(want < cap ? want : cap);
  bmoe::route_rows_kernel<<<grid, bmoe::kRouteThreads, 0, static_cast<cudaStream_t>(stream)>>>(a);
  return cudaPeekAtLastError() == cudaSuccess ? BMOE_OK : BMOE_CUDA_ERROR;
}

// Buffers other processes of the node can map (CUDA IPC over NVLink peers).
extern "C" int bmoe_peer_alloc(uint64_t bytes, void** ptr_out, uint8_t* handle_out) {
  if (ptr_out == nullptr || handle_out == nullptr || bytes == 0) return BMOE_INVALID_ARGUMENT;
  void* p = nullptr;
  if (cudaMalloc(&p, bytes) != cudaSuccess) return BMOE_CUDA_ERROR;
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, p) != cudaSuccess) {
    cudaFree(p);
    return BMOE_CUDA_ERROR;
  }
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  memcpy(handle_out, &h, 64);
  *ptr_out = p;
  return BMOE_OK;
}

extern "C" int bmoe_peer_open(const uint8_t* handle, void** ptr_out) {
  if (handle == nullptr || ptr_out == nullptr) return BMOE_INVALID_ARGUMENT;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, 64);
  void* p = nullptr;
  if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
    return BMOE_CUDA_ERROR;
  }
  *ptr_out = p;
  return BMOE_OK;
}

extern "C" int bmoe_peer_close(void* ptr) {
  if (ptr == nullptr) return BMOE_OK;
  return cudaIpcCloseMemHandle(ptr) == cudaSuccess ? BMOE_OK : BMOE_CUDA_ERROR;
}

extern "C" int bmoe_peer_free(void* ptr) {
  if (ptr == nullptr) return BMOE_OK;
  return cudaFree(ptr) == cudaSuccess ? BMOE_OK : BMOE_CUDA_ERROR;
}
