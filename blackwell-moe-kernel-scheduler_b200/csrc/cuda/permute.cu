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
#include "preload.cuh"

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
  const uint64_t resident = 16ull * bmoe::device_sm_count();
  const uint32_t grid = static_cast<uint32_t>(want < resident ? want : resident);
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
  uint64_t cap = max_ctas != 0 ? max_ctas : 8ull * bmoe::device_sm_count();
  const uint32_t grid = static_cast<uint32_t>(want < cap ? want : cap);
  bmoe::route_rows_kernel<<<grid, bmoe::kRouteThreads, 0, static_cast<cudaStream_t>(stream)>>>(a);
  return cudaPeekAtLastError() == cudaSuccess ? BMOE_OK : BMOE_CUDA_ERROR;
}

// ------------------------------------------------------------------------
// Weighted top-k combine (the un-permute after the expert GEMMs):
//   out[t, :] = bf16( sum_j weight[t, j] * float(src[rank[t, j]][row[t, j], :]) )
// FP32 accumulation with one fused multiply-add per term, j ascending, one BF16
// rounding at the end. Source rows may live on other GPUs of the node (peer
// pointers), which fuses the combine exchange with the reduction: every result
// row crosses NVLink once and is never staged in local memory. HBM / NVLink
// bound: (top_k + 1) * n * 2 bytes per token.
// ------------------------------------------------------------------------
namespace bmoe {
namespace {

constexpr uint32_t kCombineThreads = 256;
constexpr uint32_t kCombineLoads = 8;  // 16-byte loads in flight per lane

struct CombineArgs {
  const uint4* const* src_bases;  // [n_src]
  const int32_t* src_rank;        // [tokens * top_k] or nullptr (src_bases[0])
  const int64_t* src_row;         // [tokens * top_k]; negative = dropped assignment
  const float* weights;           // [tokens * top_k] or nullptr (all 1.0f)
  uint4* out;                     // [tokens, n] BF16
  uint64_t tokens;
  uint32_t top_k;
  uint32_t vec_per_row;           // n / 8
  uint32_t n_src;
  uint64_t src_rows_cap;
};

__device__ __forceinline__ void fma_bf16x8(float (&acc)[8], const uint4& v, float w) {
  const uint32_t words[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    acc[2 * i] = fmaf(w, __uint_as_float(words[i] << 16), acc[2 * i]);
    acc[2 * i + 1] = fmaf(w, __uint_as_float(words[i] & 0xffff0000u), acc[2 * i + 1]);
  }
}

__device__ __forceinline__ uint32_t pack2_bf16_rn(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

// One warp per (token, chunk of 32 * V vectors): a lane owns V vectors of the
// chunk (32 lanes apart, so every load instruction is one contiguous 512 bytes)
// and keeps kCombineLoads loads in flight: U = kCombineLoads / V source rows at a
// time. Small top_k takes the wide variants. Lane u of each group of U loads the
// routing entry (row, rank, weight) of term j0 + u; the warp shares it by shuffle.
template <uint32_t V>
__global__ void __launch_bounds__(kCombineThreads, 3) combine_topk_kernel(CombineArgs a) {
  constexpr uint32_t U = kCombineLoads / V;
  const uint32_t lane = threadIdx.x & 31;
  const uint32_t chunks = (a.vec_per_row + 32 * V - 1) / (32 * V);
  const uint64_t items = a.tokens * chunks;
  const uint64_t warps = static_cast<uint64_t>(gridDim.x) * (kCombineThreads / 32);
  for (uint64_t item = static_cast<uint64_t>(blockIdx.x) * (kCombineThreads / 32) +
                       (threadIdx.x >> 5);
       item < items; item += warps) {
    const uint64_t t = item / chunks;
    const uint32_t v0 = static_cast<uint32_t>(item % chunks) * 32 * V + lane;
    float acc[V][8];
#pragma unroll
    for (uint32_t x = 0; x < V; ++x) {
#pragma unroll
      for (uint32_t i = 0; i < 8; ++i) acc[x][i] = 0.f;
    }
    for (uint32_t j0 = 0; j0 < a.top_k; j0 += U) {
      // routing entry of term j0 + (lane % U)
      const uint32_t my_j = j0 + lane % U;
      long long my_row = -1;
      int my_rank = 0;
      float my_w = 0.f;
      if (my_j < a.top_k) {
        const uint64_t slot = t * a.top_k + my_j;
        my_row = a.src_row[slot];
        my_rank = a.src_rank != nullptr ? a.src_rank[slot] : 0;
        my_w = a.weights != nullptr ? a.weights[slot] : 1.0f;
        // Dropped or out-of-range assignments contribute nothing and touch no memory.
        if (my_row < 0 || static_cast<uint64_t>(my_row) >= a.src_rows_cap || my_rank < 0 ||
            static_cast<uint32_t>(my_rank) >= a.n_src) {
          my_row = -1;
        }
      }
      uint4 regs[U][V];
      float w[U];
      bool live[U];
#pragma unroll
      for (uint32_t u = 0; u < U; ++u) {
        const long long row = __shfl_sync(0xffffffffu, my_row, u);
        const int rank = __shfl_sync(0xffffffffu, my_rank, u);
        w[u] = __shfl_sync(0xffffffffu, my_w, u);
        const uint4* base =
            row >= 0 ? a.src_bases[rank] + static_cast<uint64_t>(row) * a.vec_per_row : nullptr;
#pragma unroll
        for (uint32_t x = 0; x < V; ++x) {
          const uint32_t v = v0 + 32 * x;
          regs[u][x] = (base != nullptr && v < a.vec_per_row) ? base[v] : make_uint4(0u, 0u, 0u, 0u);
        }
        live[u] = row >= 0;
      }
      // Terms in ascending j; dropped terms are skipped, not multiplied by zero.
#pragma unroll
      for (uint32_t u = 0; u < U; ++u) {
        if (live[u]) {
#pragma unroll
          for (uint32_t x = 0; x < V; ++x) fma_bf16x8(acc[x], regs[u][x], w[u]);
        }
      }
    }
#pragma unroll
    for (uint32_t x = 0; x < V; ++x) {
      const uint32_t v = v0 + 32 * x;
      if (v < a.vec_per_row) {
        a.out[t * a.vec_per_row + v] = make_uint4(
            pack2_bf16_rn(acc[x][0], acc[x][1]), pack2_bf16_rn(acc[x][2], acc[x][3]),
            pack2_bf16_rn(acc[x][4], acc[x][5]), pack2_bf16_rn(acc[x][6], acc[x][7]));
      }
    }
  }
}

// CTAs of `kernel` that fit the device at once (grid-stride kernels launch no more).
template <typename Kernel>
uint32_t resident_ctas(Kernel kernel, int threads) {
  int device = 0, sms = 0, per_sm = 0;
  if (cudaGetDevice(&device) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess ||
      cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, 0) != cudaSuccess ||
      sms <= 0 || per_sm <= 0) {
    return 148u * 4u;
  }
  return static_cast<uint32_t>(sms) * static_cast<uint32_t>(per_sm);
}

}  // namespace
}  // namespace bmoe

extern "C" int bmoe_combine_topk(const void* const* src_bases_dev, uint32_t n_src,
                                 uint64_t src_rows_cap, const int32_t* src_rank_dev,
                                 const int64_t* src_row_dev, const float* weights_dev,
                                 uint64_t tokens, uint32_t top_k, uint32_t n,
                                 void* out_dev, uint32_t max_ctas, void* stream) {
  if (tokens == 0) return BMOE_OK;
  if (src_bases_dev == nullptr || n_src == 0 || src_row_dev == nullptr || out_dev == nullptr ||
      top_k == 0 || n == 0 || n % 8 != 0 ||
      (reinterpret_cast<uintptr_t>(out_dev) & 15u) != 0) {
    return BMOE_INVALID_ARGUMENT;
  }
  bmoe::CombineArgs a;
  a.src_bases = reinterpret_cast<const uint4* const*>(src_bases_dev);
  a.src_rank = src_rank_dev;
  a.src_row = src_row_dev;
  a.weights = weights_dev;
  a.out = static_cast<uint4*>(out_dev);
  a.tokens = tokens;
  a.top_k = top_k;
  a.vec_per_row = n / 8;
  a.n_src = n_src;
  a.src_rows_cap = src_rows_cap;
  // Vectors per lane: 4 (a warp reads 2 KB contiguous of every source row, which
  // measured 5.7-6.1 TB/s against 3.3 TB/s for 512-byte pieces), less only when
  // the row is narrower.
  uint32_t v = 4;
  while (v > 1 && 32u * v > a.vec_per_row) v >>= 1;
  const uint64_t chunks = (a.vec_per_row + 32ull * v - 1) / (32ull * v);
  const uint64_t want = (tokens * chunks + 7) / 8;
  auto launch = [&](auto kernel) {
    static const uint32_t resident = bmoe::resident_ctas(kernel, bmoe::kCombineThreads);
    const uint64_t cap = max_ctas != 0 ? max_ctas : resident;
    const uint32_t grid = static_cast<uint32_t>(want < cap ? want : cap);
    kernel<<<grid, bmoe::kCombineThreads, 0, static_cast<cudaStream_t>(stream)>>>(a);
  };
  switch (v) {
    case 1: launch(bmoe::combine_topk_kernel<1>); break;
    case 2: launch(bmoe::combine_topk_kernel<2>); break;
    default: launch(bmoe::combine_topk_kernel<4>); break;
  }
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

namespace bmoe {
cudaError_t preload_permute_kernels() {
  cudaError_t rc = preload_one(gather_rows_kernel);
  if (rc == cudaSuccess) rc = preload_one(route_rows_kernel);
  if (rc == cudaSuccess) rc = preload_one(combine_topk_kernel<1>);
  if (rc == cudaSuccess) rc = preload_one(combine_topk_kernel<2>);
  if (rc == cudaSuccess) rc = preload_one(combine_topk_kernel<4>);
  return rc;
}
}  // namespace bmoe
