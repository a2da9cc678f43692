// On-device worklist builder: integer kernels that turn per-expert token counts
// into the tile worklist the grouped-GEMM kernel walks.
//
//   plan kernel   (1 CTA)  per-expert tile counts, exclusive prefix sums (row
//                          offsets, tile offsets), ascending active-expert
//                          compaction, and the visiting order of experts:
//                          identity, or stable descending by tile count
//   expand kernel (grid)   one thread per tile record: binary search of the
//                          visit-order tile prefix, then (tile_m, tile_n) from
//                          the position inside the expert's tile grid
//
// Output records are byte-identical to the reference host scheduler:
//   build_expert_tiles                  src/scheduler/scheduler.cpp:37-60
//   order_by_descending_expert_tiles    src/scheduler/scheduler.cpp:80-103
// and the active-expert list equals the host filter of the reference plan
// (baselines/cutlass/cutlass_baseline.cu:243-266).
#include <cuda_runtime.h>

#include <atomic>

#include <cstdint>

#include "bmoe_b200.h"
#include "preload.cuh"

namespace bmoe {

namespace {

constexpr uint32_t kPlanThreads = 1024;
constexpr uint32_t kExpandThreads = 256;

struct WorklistArrays {
  bmoe_worklist_totals* totals;
  uint64_t* row_offsets;
  uint32_t* expert_m_tiles;
  uint32_t* expert_tiles;
  uint32_t* tile_offsets;
  uint32_t* active_ids;
  uint32_t* visit_order;
  uint32_t* visit_tile_offsets;
};

__device__ __forceinline__ uint32_t ceil_div_u32(uint32_t a, uint32_t b) {
  return a == 0 ? 0 : (a - 1) / b + 1;
}

// Block-wide exclusive scan of one value per thread; returns the exclusive
// prefix and leaves the block total in *total. `scratch` holds 32 entries.
__device__ uint64_t block_exclusive_scan(uint64_t value, uint64_t* scratch,
                                         uint64_t* total) {
  const uint32_t lane = threadIdx.x & 31;
  const uint32_t warp = threadIdx.x >> 5;
  uint64_t inclusive = value;
#pragma unroll
  for (uint32_t d = 1; d < 32; d <<= 1) {
    const uint64_t up = __shfl_up_sync(0xffffffffu, inclusive, d);
    if (lane >= d) inclusive += up;
  }
  if (lane == 31) scratch[warp] = inclusive;
  __syncthreads();
  if (warp == 0) {
    uint64_t w = lane < (blockDim.x >> 5) ? scratch[lane] : 0;
#pragma unroll
    for (uint32_t d = 1; d < 32; d <<= 1) {
      const uint64_t up = __shfl_up_sync(0xffffffffu, w, d);
      if (lane >= d) w += up;
    }
    scratch[lane] = w;  // inclusive warp totals
  }
  __syncthreads();
  const uint64_t warp_base = warp == 0 ? 0 : scratch[warp - 1];
  *total = scratch[(blockDim.x >> 5) - 1];
  __syncthreads();
  return warp_base + inclusive - value;
}

__global__ void __launch_bounds__(kPlanThreads)
worklist_plan_kernel(const uint32_t* __restrict__ counts, bmoe_worklist_request req,
                     uint32_t tile_capacity, WorklistArrays out) {
  __shared__ uint64_t scratch[32];
  const uint32_t experts = req.experts;
  const uint32_t n_tiles = (req.n + req.tile_n - 1) / req.tile_n;

  // Pass 1: per-expert tile counts and the three prefix sums, in chunks of
  // blockDim.x experts with running carries.
  uint64_t row_carry = 0, tile_carry = 0, active_carry = 0;
  for (uint32_t chunk = 0; chunk < experts; chunk += blockDim.x) {
    const uint32_t e = chunk + threadIdx.x;
    const bool in_range = e < experts;
    const uint32_t rows = in_range ? counts[e] : 0;
    const uint32_t m_tiles = ceil_div_u32(rows, req.tile_m);
    const uint64_t tiles = static_cast<uint64_t>(m_tiles) * n_tiles;
    const uint64_t is_active = rows != 0 ? 1 : 0;

    uint64_t row_total, tile_total, active_total;
    const uint64_t row_prefix = block_exclusive_scan(rows, scratch, &row_total);
    const uint64_t tile_prefix = block_exclusive_scan(tiles, scratch, &tile_total);
    const uint64_t active_prefix =
        block_exclusive_scan(is_active, scratch, &active_total);
    if (in_range) {
      out.expert_m_tiles[e] = m_tiles;
      out.expert_tiles[e] = static_cast<uint32_t>(tiles);
      out.row_offsets[e] = row_carry + row_prefix;
      out.tile_offsets[e] = static_cast<uint32_t>(tile_carry + tile_prefix);
      if (is_active) {
        out.active_ids[active_carry + active_prefix] = e;
      }
    }
    row_carry += row_total;
    tile_carry += tile_total;
    active_carry += active_total;
  }
  for (uint32_t i = static_cast<uint32_t>(active_carry) + threadIdx.x; i < experts;
       i += blockDim.x) {
    out.active_ids[i] = 0xffffffffu;
  }
  if (threadIdx.x == 0) {
    out.row_offsets[experts] = row_carry;
    out.tile_offsets[experts] = static_cast<uint32_t>(tile_carry);
    out.totals->total_tiles = static_cast<uint32_t>(tile_carry);
    out.totals->active_experts = static_cast<uint32_t>(active_carry);
    out.totals->total_rows = row_carry;
    out.totals->total_valid_elements = row_carry * req.n;
    out.totals->overflow =
        (tile_carry > 0xffffffffull || tile_carry > tile_capacity) ? 1u : 0u;
    out.totals->reserved = 0;
  }
  __syncthreads();

  // Pass 2: visiting order. Position of expert e = number of experts that come
  // before it under (more tiles first, then lower id): a stable descending
  // sort written as a rank computation.
  for (uint32_t e = threadIdx.x; e < experts; e += blockDim.x) {
    uint32_t position = e;
    if (req.order == BMOE_ORDER_SORTED_BY_WORK) {
      const uint32_t mine = out.expert_tiles[e];
      position = 0;
      for (uint32_t j = 0; j < experts; ++j) {
        const uint32_t theirs = out.expert_tiles[j];
        position += (theirs > mine || (theirs == mine && j < e)) ? 1u : 0u;
      }
    }
    out.visit_order[position] = e;
  }
  __syncthreads();

  // Pass 3: exclusive prefix of tile counts in visiting order.
  uint64_t carry = 0;
  for (uint32_t chunk = 0; chunk < experts; chunk += blockDim.x) {
    const uint32_t pos = chunk + threadIdx.x;
    const uint64_t tiles = pos < experts ? out.expert_tiles[out.visit_order[pos]] : 0;
    uint64_t total;
    const uint64_t prefix = block_exclusive_scan(tiles, scratch, &total);
    if (pos < experts) {
      out.visit_tile_offsets[pos] = static_cast<uint32_t>(carry + prefix);
    }
    carry += total;
  }
  if (threadIdx.x == 0) {
    out.visit_tile_offsets[experts] = static_cast<uint32_t>(carry);
  }
}

__global__ void __launch_bounds__(kExpandThreads)
worklist_expand_kernel(const uint32_t* __restrict__ counts, bmoe_worklist_request req,
                       bmoe_tile* __restrict__ tiles, uint32_t tile_capacity,
                       WorklistArrays arrays) {
  const uint32_t experts = req.experts;
  const uint32_t n_tiles = (req.n + req.tile_n - 1) / req.tile_n;
  const uint32_t total = min(arrays.totals->total_tiles, tile_capacity);
  const uint32_t* __restrict__ prefix = arrays.visit_tile_offsets;

  for (uint32_t t = blockIdx.x * blockDim.x + threadIdx.x; t < total;
       t += gridDim.x * blockDim.x) {
    // Largest position whose prefix is <= t (positions without tiles share a
    // prefix value with their successor and are skipped by taking the last).
    uint32_t lo = 0, hi = experts;
    while (hi - lo > 1) {
      const uint32_t mid = (lo + hi) >> 1;
      if (prefix[mid] <= t) lo = mid; else hi = mid;
    }
    const uint32_t expert = arrays.visit_order[lo];
    const uint32_t local = t - prefix[lo];
    const uint32_t rows = counts[expert];
    const uint32_t m_tiles = arrays.expert_m_tiles[expert];
    uint32_t tm, tn;
    if (req.raster == BMOE_RASTER_M_FASTEST) {
      tn = local / m_tiles;
      tm = local - tn * m_tiles;
    } else {
      tm = local / n_tiles;
      tn = local - tm * n_tiles;
    }
    bmoe_tile rec;
    rec.expert_id = expert;
    rec.tile_m = tm;
    rec.tile_n = tn;
    rec.valid_m = min(req.tile_m, rows - tm * req.tile_m);
    rec.valid_n = min(req.tile_n, req.n - tn * req.tile_n);
    tiles[t] = rec;
  }
}

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

}  // namespace

}  // namespace bmoe

extern "C" {

int bmoe_worklist_layout_for(uint32_t experts, bmoe_worklist_layout* out) {
  if (out == nullptr || experts == 0 || experts > BMOE_WORKLIST_MAX_EXPERTS) {
    return BMOE_INVALID_ARGUMENT;
  }
  size_t cursor = 0;
  auto take = [&cursor](size_t bytes) {
    const size_t at = cursor;
    cursor = bmoe::align_up(cursor + bytes, 256);
    return at;
  };
  const size_t e = experts;
  out->off_totals = take(sizeof(bmoe_worklist_totals));
  out->off_row_offsets = take(sizeof(uint64_t) * (e + 1));
  out->off_expert_m_tiles = take(sizeof(uint32_t) * e);
  out->off_expert_tiles = take(sizeof(uint32_t) * e);
  out->off_tile_offsets = take(sizeof(uint32_t) * (e + 1));
  out->off_active_ids = take(sizeof(uint32_t) * e);
  out->off_visit_order = take(sizeof(uint32_t) * e);
  out->off_visit_tile_offsets = take(sizeof(uint32_t) * (e + 1));
  out->bytes = cursor;
  return BMOE_OK;
}

int bmoe_worklist_build(const uint32_t* counts_dev,
                        const bmoe_worklist_request* request,
                        bmoe_tile* tiles_dev, uint32_t tile_capacity,
                        void* workspace_dev, void* stream) {
  if (counts_dev == nullptr || request == nullptr || workspace_dev == nullptr ||
      (tiles_dev == nullptr && tile_capacity != 0)) {
    return BMOE_INVALID_ARGUMENT;
  }
  if (request->tile_m == 0 || request->tile_n == 0 || request->order > 1 ||
      request->raster > 1 ||
      (reinterpret_cast<uintptr_t>(workspace_dev) & 255u) != 0) {
    return BMOE_INVALID_ARGUMENT;
  }
  // The sorted order ranks every expert against every other one inside one CTA
  // (experts^2 / 1024 steps per thread): bounded so that it stays tens of microseconds.
  if (request->order == BMOE_ORDER_SORTED_BY_WORK &&
      request->experts > BMOE_WORKLIST_MAX_SORTED_EXPERTS) {
    return BMOE_INVALID_ARGUMENT;
  }
  bmoe_worklist_layout layout;
  const int rc = bmoe_worklist_layout_for(request->experts, &layout);
  if (rc != BMOE_OK) return rc;

  uint8_t* const ws = static_cast<uint8_t*>(workspace_dev);
  bmoe::WorklistArrays arrays;
  arrays.totals = reinterpret_cast<bmoe_worklist_totals*>(ws + layout.off_totals);
  arrays.row_offsets = reinterpret_cast<uint64_t*>(ws + layout.off_row_offsets);
  arrays.expert_m_tiles = reinterpret_cast<uint32_t*>(ws + layout.off_expert_m_tiles);
  arrays.expert_tiles = reinterpret_cast<uint32_t*>(ws + layout.off_expert_tiles);
  arrays.tile_offsets = reinterpret_cast<uint32_t*>(ws + layout.off_tile_offsets);
  arrays.active_ids = reinterpret_cast<uint32_t*>(ws + layout.off_active_ids);
  arrays.visit_order = reinterpret_cast<uint32_t*>(ws + layout.off_visit_order);
  arrays.visit_tile_offsets =
      reinterpret_cast<uint32_t*>(ws + layout.off_visit_tile_offsets);

  cudaStream_t s = static_cast<cudaStream_t>(stream);
  bmoe::worklist_plan_kernel<<<1, bmoe::kPlanThreads, 0, s>>>(
      counts_dev, *request, tile_capacity, arrays);
  if (cudaPeekAtLastError() != cudaSuccess) return BMOE_CUDA_ERROR;
  if (tile_capacity != 0) {
    // The tile total is only known on the device; a fixed grid strides over it.
    const uint32_t want = (tile_capacity + bmoe::kExpandThreads - 1) / bmoe::kExpandThreads;
    const uint32_t resident = 8u * bmoe::device_sm_count();
    const uint32_t grid = want < resident ? want : resident;
    bmoe::worklist_expand_kernel<<<grid, bmoe::kExpandThreads, 0, s>>>(
        counts_dev, *request, tiles_dev, tile_capacity, arrays);
    if (cudaPeekAtLastError() != cudaSuccess) return BMOE_CUDA_ERROR;
  }
  return BMOE_OK;
}

}  // extern "C"

// ------------------------------------------------------------------------
// Allocation-free variant: the auxiliary arrays live in the library image.
// ------------------------------------------------------------------------
namespace bmoe {
namespace {

// Room for bmoe_worklist_layout_for(BMOE_WORKLIST_STATIC_MAX_EXPERTS): 33792
// bytes, rounded up. Every GPU that loads the library holds this until exit.
constexpr size_t kStaticScratchBytes = 34 * 1024;
static __device__ __align__(256) unsigned char g_worklist_scratch[kStaticScratchBytes];

// In host code `g_worklist_scratch` is only a handle for the runtime, not a
// device address; the address is looked up once per device, with that device
// current, and cached here.
constexpr int kMaxDevices = 64;
// Two host threads may resolve the address at the same time; both store the same
// value, and the atomic makes that a defined program.
std::atomic<void*> g_scratch_address[kMaxDevices];

// Device address of the array on the current device (looked up on first use).
void* static_scratch_address() {
  int device = -1;
  if (cudaGetDevice(&device) != cudaSuccess) return nullptr;
  if (device < 0 || device >= kMaxDevices) return nullptr;
  void* address = g_scratch_address[device].load(std::memory_order_acquire);
  if (address == nullptr) {
    if (cudaGetSymbolAddress(&address, g_worklist_scratch) != cudaSuccess) return nullptr;
    g_scratch_address[device].store(address, std::memory_order_release);
  }
  return address;
}

}  // namespace
}  // namespace bmoe

extern "C" int bmoe_worklist_build_static(const uint32_t* counts_dev,
                                          const bmoe_worklist_request* request,
                                          bmoe_tile* tiles_dev, uint32_t tile_capacity,
                                          bmoe_worklist_totals* totals_out_dev,
                                          void* stream) {
  if (request == nullptr || request->experts == 0 ||
      request->experts > BMOE_WORKLIST_STATIC_MAX_EXPERTS) {
    return BMOE_INVALID_ARGUMENT;  // beyond what the fixed array can hold
  }
  bmoe_worklist_layout layout;
  if (bmoe_worklist_layout_for(request->experts, &layout) != BMOE_OK ||
      layout.bytes > bmoe::kStaticScratchBytes) {
    return BMOE_INVALID_ARGUMENT;
  }
  // First use on this device resolves the address (keep it outside stream capture;
  // bmoe_preload_kernels does it too).
  void* const scratch = bmoe::static_scratch_address();
  if (scratch == nullptr) return BMOE_CUDA_ERROR;
  // The planning kernel writes every array element and every totals field it
  // or the expansion kernel later reads, so nothing needs clearing here.
  const int rc = bmoe_worklist_build(counts_dev, request, tiles_dev, tile_capacity,
                                     scratch, stream);
  if (rc != BMOE_OK) return rc;
  if (totals_out_dev != nullptr) {
    const void* totals = static_cast<const unsigned char*>(scratch) + layout.off_totals;
    if (cudaMemcpyAsync(totals_out_dev, totals, sizeof(bmoe_worklist_totals),
                        cudaMemcpyDeviceToDevice,
                        static_cast<cudaStream_t>(stream)) != cudaSuccess) {
      return BMOE_CUDA_ERROR;
    }
  }
  return BMOE_OK;
}

namespace bmoe {
cudaError_t preload_worklist_kernels() {
  cudaError_t rc = preload_one(worklist_plan_kernel);
  if (rc == cudaSuccess) rc = preload_one(worklist_expand_kernel);
  // Also resolve the fixed array of the allocation-free entry point, so that a caller
  // that preloads has nothing left to do before a stream capture.
  if (rc == cudaSuccess && static_scratch_address() == nullptr) rc = cudaErrorUnknown;
  return rc;
}
}  // namespace bmoe
