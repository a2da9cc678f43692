// C interface, device half: the grouped-GEMM plan (section 3 of bmoe_b200.h).
//
// initialize() does everything that can be prepared ahead of a launch: argument
// checks, policy resolution, host encoding of one TMA descriptor triple per
// active expert, ONE asynchronous copy (from pinned staging memory) of counts,
// descriptors, queue and status words, and the on-device worklist build. It
// enqueues on the plan's stream and does not wait for the device; a plan must
// not be re-initialised while launches of it are still in flight on ANOTHER
// stream. run() is a single kernel launch. Behavioural contract
// (status codes, null / zero handling, stream override) follows
// baselines/cutlass/cutlass_baseline.cu:195-377 of the reference.
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>
#include <cstring>
#include <new>
#include <vector>

#include "blackwell_moe/dispatch.hpp"
#include "bmoe_b200.h"
#include "gemm_sm100.cuh"
#include "preload.cuh"

namespace {

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*,
                                   const cuuint32_t*, const cuuint32_t*,
                                   CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// cuTensorMapEncodeTiled is resolved through the runtime so the library has no
// link-time dependency on libcuda.
EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = []() -> EncodeTiledFn {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult query = cudaDriverEntryPointSymbolNotFound;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault,
                                &query) != cudaSuccess ||
        query != cudaDriverEntryPointSuccess) {
      return nullptr;
    }
    return reinterpret_cast<EncodeTiledFn>(sym);
  }();
  return fn;
}

// Element type of a matrix a tensor map describes.
enum class Elem : uint32_t { kBf16, kF32, kByte };

// Row-major matrix [rows, cols] viewed as a 2-D tensor {cols, rows} with a SWIZZLE_128B
// box of 128 bytes (64 BF16 / 32 FP32 / 128 one-byte columns) x box_rows rows.
bool encode_matrix(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols,
                   uint32_t box_rows, Elem type) {
  EncodeTiledFn encode = encode_tiled_fn();
  if (encode == nullptr) return false;
  const uint32_t elem = type == Elem::kF32 ? 4u : (type == Elem::kBf16 ? 2u : 1u);
  const CUtensorMapDataType kind =
      type == Elem::kF32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                         : (type == Elem::kBf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                : CU_TENSOR_MAP_DATA_TYPE_UINT8);
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {cols * elem};
  const cuuint32_t box[2] = {128u / elem, box_rows};
  const cuuint32_t elem_strides[2] = {1, 1};
  const CUresult rc = encode(
      map, kind, 2, const_cast<void*>(base), dims, strides,
      box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
      CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return rc == CUDA_SUCCESS;
}

// Grow-only device allocation.
struct DeviceBlock {
  void* ptr = nullptr;
  size_t bytes = 0;
  bool reserve(size_t want) {
    if (want <= bytes) return true;
    release();
    if (cudaMalloc(&ptr, want) != cudaSuccess) {
      ptr = nullptr;
      return false;
    }
    bytes = want;
    return true;
  }
  void release() {
    if (ptr != nullptr) cudaFree(ptr);
    ptr = nullptr;
    bytes = 0;
  }
};

// Grow-only pinned host staging area (asynchronous H2D copies need it).
struct PinnedBlock {
  void* ptr = nullptr;
  size_t bytes = 0;
  bool reserve(size_t want) {
    if (want <= bytes) return true;
    release();
    if (cudaHostAlloc(&ptr, want, cudaHostAllocDefault) != cudaSuccess) {
      ptr = nullptr;
      return false;
    }
    bytes = want;
    return true;
  }
  void release() {
    if (ptr != nullptr) cudaFreeHost(ptr);
    ptr = nullptr;
    bytes = 0;
  }
};

bool misaligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) != 0; }

}  // namespace

struct bmoe_plan {
  bool ready = false;
  bmoe_plan_stats stats{};
  cudaStream_t default_stream = nullptr;
  cudaStream_t setup_stream = nullptr;
  cudaStream_t last_stream = nullptr;
  cudaEvent_t setup_done = nullptr;
  int device = -1;

  // One metadata block, filled by a single copy from pinned staging memory:
  //   [0, 256) queue words   [256, 512) DeviceStatus
  //   [512, ...) counts uint32 [experts]   then CUtensorMap [3][experts] (128-aligned)
  DeviceBlock meta;
  PinnedBlock staging;
  DeviceBlock worklist;   // bmoe_tile [capacity]
  DeviceBlock workspace;  // worklist builder arrays

  // What the B descriptors in the staging area were encoded for (reused while the
  // expert's weight pointer, the shape and the box do not change).
  std::vector<const void*> b_encoded_for;
  uint32_t b_key_n = 0, b_key_k = 0, b_key_box = 0, b_key_experts = 0, b_key_type = 0;
  bool needs_push = false;   // results_pushed: run() only after set_push

  bmoe::GemmParams params{};
  uint32_t units = 0;      // persistent CTAs or CTA pairs (tile count for CLC)
  uint32_t tile_n = 0;
  uint32_t stats_n = 0;    // output columns of the current problem
  uint32_t cta_group = 1;
  bool out_f32 = false;

  void release_all() {
    meta.release();
    staging.release();
    b_encoded_for.clear();
    worklist.release();
    workspace.release();
    if (setup_done != nullptr) cudaEventDestroy(setup_done);
    setup_done = nullptr;
    ready = false;
  }
};

namespace {

struct Resolved {
  uint32_t scheduler;      // policy after "auto" resolution
  uint32_t order;          // bmoe_worklist_order
  uint32_t sched_mode;     // bmoe::SchedMode
  uint32_t claim_size;
  uint32_t tail_tiles;
  bool one_cta_per_tile;
};

Resolved resolve_policy(const bmoe_gemm_args& a, uint32_t tile_m, uint32_t tile_n,
                        uint32_t cta_count) {
  Resolved r{};
  r.scheduler = a.scheduler;
  r.order = BMOE_ORDER_EXPERT;
  r.sched_mode = bmoe::kSchedStatic;
  r.claim_size = 1;
  r.tail_tiles = 0;
  r.one_cta_per_tile = false;

  uint32_t policy = a.scheduler;
  uint32_t claim = a.claim_size == 0 ? 1 : a.claim_size;
  uint32_t tail = a.hybrid_tail_tiles;
  if (policy == BMOE_SCHED_AUTO) {
    // Dispatch on launch-level routing features with the rule fitted on this engine
    // (the reference's rule and bootstrap values stay available through
    // select_launch_variant / bmoe_select_variant).
    namespace bm = blackwell_moe;
    bm::GemmShape shape;
    shape.n = a.n;
    shape.k = a.k;
    shape.tile_m = tile_m;
    shape.tile_n = tile_n;
    const std::vector<uint32_t> counts(a.tokens_per_expert,
                                       a.tokens_per_expert + a.experts);
    const bm::RoutingFeatures f = bm::routing_features(counts, shape, cta_count);
    bm::DispatchSpec spec;
    spec.cta_count = cta_count;
    // The tail is two waves of the persistent grid, as in the reference spec
    // (296 = 2 x 148).
    spec.hybrid_tail_tiles = 2 * cta_count;
    const bm::LaunchConfig cfg =
        bm::resolve_launch_config(
            bm::select_launch_variant_fitted(f), spec);
    policy = static_cast<uint32_t>(cfg.scheduler);
    claim = cfg.claim_size;
    tail = cfg.hybrid_tail_tiles;
    r.one_cta_per_tile = cfg.one_cta_per_tile;
    r.scheduler = policy;
  }
  switch (policy) {
    case BMOE_SCHED_EXPERT_ORDER:
    case BMOE_SCHED_COMPACTED:
      break;
    case BMOE_SCHED_STATIC_PERSISTENT:
      r.order = BMOE_ORDER_SORTED_BY_WORK;
      break;
    case BMOE_SCHED_DYNAMIC_QUEUE:
      r.sched_mode = bmoe::kSchedQueue;
      r.claim_size = claim;
      r.tail_tiles = tail;
      break;
    case BMOE_SCHED_CLC:
      r.sched_mode = bmoe::kSchedClc;
      r.one_cta_per_tile = true;
      break;
    default:
      break;
  }
  return r;
}

}  // namespace

extern "C" {

bmoe_plan* bmoe_plan_create(void) { return new (std::nothrow) bmoe_plan; }

void bmoe_plan_destroy(bmoe_plan* plan) {
  if (plan == nullptr) return;
  plan->release_all();
  delete plan;
}

int bmoe_plan_initialize(bmoe_plan* plan, const bmoe_gemm_args* args) {
  if (plan == nullptr || args == nullptr) return BMOE_INVALID_ARGUMENT;
  plan->ready = false;
  plan->stats = bmoe_plan_stats{};
  const bmoe_gemm_args& a = *args;

  // ---- argument checks, in the reference's order ----
  const bool packed = a.packed_a != nullptr;
  const bool pushed = a.results_pushed != 0;
  const bool dev_counts = a.tokens_per_expert_dev != nullptr;
  if ((a.a == nullptr && !packed) || a.b == nullptr || (a.d == nullptr && !pushed) ||
      (a.tokens_per_expert == nullptr && !dev_counts) || a.experts == 0 || a.n == 0 ||
      a.k == 0 || a.n % 8 != 0 || a.k % 8 != 0) {
    return BMOE_INVALID_ARGUMENT;
  }
  // counts that the host never sees: everything that is sized from them uses capacities
  if (dev_counts && (!packed || !pushed || a.hybrid_tail_tiles != 0 ||
                     (a.scheduler != BMOE_SCHED_EXPERT_ORDER &&
                      a.scheduler != BMOE_SCHED_STATIC_PERSISTENT &&
                      a.scheduler != BMOE_SCHED_COMPACTED &&
                      a.scheduler != BMOE_SCHED_DYNAMIC_QUEUE))) {
    return BMOE_INVALID_ARGUMENT;
  }
  if (packed && (misaligned16(a.packed_a) || a.packed_rows == 0)) return BMOE_INVALID_ARGUMENT;
  if (pushed && a.output_f32 != 0) return BMOE_INVALID_ARGUMENT;
  if (a.data_type > 1) return BMOE_UNSUPPORTED_DATA_TYPE;
  // FP8 E4M3 operands: a row is k bytes, and a tensor map wants row strides of 16 bytes
  const bool fp8 = a.data_type == 1;
  if (fp8 && a.k % 16 != 0) return BMOE_INVALID_ARGUMENT;
  const Elem operand = fp8 ? Elem::kByte : Elem::kBf16;
  if (a.scheduler > BMOE_SCHED_CLC) return BMOE_UNSUPPORTED_SCHEDULER;
  if (a.experts > BMOE_WORKLIST_MAX_EXPERTS) return BMOE_INVALID_ARGUMENT;
  if (a.tile_n != 0 && a.tile_n != 64 && a.tile_n != 128 && a.tile_n != 256) {
    return BMOE_INVALID_ARGUMENT;
  }
  if (a.cta_group > 2) return BMOE_INVALID_ARGUMENT;
  // CTA pairs compute 256 x 256 tiles; a narrower tile has no pair variant.
  if (a.cta_group == 2 && a.tile_n != 0 && a.tile_n != 256) return BMOE_INVALID_ARGUMENT;

  int device = 0, major = 0, minor = 0, sm_count = 0;
  if (cudaGetDevice(&device) != cudaSuccess ||
      cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device) != cudaSuccess ||
      cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, device) != cudaSuccess ||
      cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) {
    return BMOE_CUDA_ERROR;
  }
  // The kernels are built for sm_100a only (tcgen05, TMEM).
  if (major != 10 || minor != 0) return BMOE_UNSUPPORTED_DEVICE;
  if (plan->device != device) {
    plan->release_all();
    plan->device = device;
  }

  uint32_t active = 0;
  uint64_t routed_rows = 0;
  // with device-side counts every expert may turn out active: each needs its weights
  std::vector<uint32_t> assumed_rows;
  if (dev_counts) assumed_rows.assign(a.experts, 1u);
  const uint32_t* const host_counts = dev_counts ? assumed_rows.data() : a.tokens_per_expert;
  for (uint32_t e = 0; e < a.experts; ++e) {
    if (host_counts[e] == 0) continue;
    if ((!packed && (a.a[e] == nullptr || misaligned16(a.a[e]))) || a.b[e] == nullptr ||
        misaligned16(a.b[e]) || (!pushed && (a.d[e] == nullptr || misaligned16(a.d[e])))) {
      return BMOE_INVALID_ARGUMENT;
    }
    routed_rows += host_counts[e];
    ++active;
  }
  if (packed && !dev_counts && routed_rows > a.packed_rows) return BMOE_INVALID_ARGUMENT;
  plan->stats.active_experts = active;
  plan->default_stream = static_cast<cudaStream_t>(a.stream);
  plan->setup_stream = plan->default_stream;
  plan->last_stream = plan->default_stream;
  if (active == 0) {
    // A routing result without active experts is valid and launches nothing.
    plan->ready = true;
    return BMOE_OK;
  }

  // ---- engine configuration ----
  const bool out_f32 = a.output_f32 != 0;
  // FP32 epilogue: 256-wide tiles only
  if (out_f32 && a.tile_n != 0 && a.tile_n != 256) return BMOE_INVALID_ARGUMENT;
  // cta_group 0 = choose: CTA pairs (256-row tiles, a third less operand traffic
  // per FLOP) unless 256-row tiles would pad the routed rows by more than 10 %
  // over 128-row tiles, as they do for small-M (decode-like) routing.
  uint32_t cta_group = a.cta_group;
  if (cta_group == 0 && dev_counts) cta_group = a.n > 128 ? 2u : 1u;
  if (cta_group == 0) {
    uint64_t padded128 = 0, padded256 = 0;
    for (uint32_t e = 0; e < a.experts; ++e) {
      const uint64_t rows = a.tokens_per_expert[e];
      padded128 += (rows + 127) / 128 * 128;
      padded256 += (rows + 255) / 256 * 256;
    }
    const bool pair_ok = (a.tile_n == 0 || a.tile_n == 256) && a.n > 128;
    cta_group = (pair_ok && padded256 * 10 <= padded128 * 11) ? 2u : 1u;
  }
  const uint32_t tile_m = 128 * cta_group;
  uint32_t tile_n = 256u;
  if (cta_group == 1 && !out_f32) {
    if (a.tile_n != 0) {
      tile_n = a.tile_n;
    } else if (!dev_counts) {
      // More tiles than SMs: 256-column tiles (fewest operand bytes per FLOP). Fewer:
      // the launch is one wave and is bound by how many bytes of the weight stream
      // each CTA keeps in flight, so 128-column tiles are used as long as they still
      // fit one wave (twice the CTAs pulling on memory). 64-column tiles (tile_n = 64,
      // explicit only) measured no faster: twice the CTAs again, but each keeps less in
      // flight. The k order of a tile does not depend on its width, so results do not
      // change.
      const uint32_t wave = a.cta_count != 0 ? a.cta_count : static_cast<uint32_t>(sm_count);
      tile_n = 256u;
      if (bmoe_host_tile_count(a.tokens_per_expert, a.experts, a.n, tile_m, 256u) < wave &&
          bmoe_host_tile_count(a.tokens_per_expert, a.experts, a.n, tile_m, 128u) <= wave) {
        tile_n = 128u;
      }
      if (a.n <= 64) tile_n = 64u;
    }
  }
  const uint32_t raster =
      a.raster_along_m < 0 ? BMOE_RASTER_M_FASTEST
                           : (a.raster_along_m != 0 ? BMOE_RASTER_M_FASTEST
                                                    : BMOE_RASTER_N_FASTEST);
  // Scheduling units: persistent CTAs, or CTA pairs (one per two SMs).
  const uint32_t sm_units = static_cast<uint32_t>(sm_count) / cta_group;
  const uint32_t unit_budget = a.cta_count != 0 ? a.cta_count : (sm_units ? sm_units : 1u);
  const Resolved policy = resolve_policy(a, tile_m, tile_n, unit_budget);

  // device-side counts: sum(ceil(M_e / tile_m)) <= floor(rows / tile_m) + experts
  const uint64_t tile_total =
      dev_counts ? (a.packed_rows / tile_m + a.experts) * ((a.n + tile_n - 1) / tile_n)
                 : bmoe_host_tile_count(a.tokens_per_expert, a.experts, a.n, tile_m, tile_n);
  if (tile_total == 0 || tile_total > 0x7fffffffull) return BMOE_INVALID_ARGUMENT;
  const uint32_t tiles = static_cast<uint32_t>(tile_total);

  // ---- device storage ----
  bmoe_worklist_layout layout;
  if (bmoe_worklist_layout_for(a.experts, &layout) != BMOE_OK) {
    return BMOE_INVALID_ARGUMENT;
  }
  const size_t map_bytes = sizeof(CUtensorMap) * 3 * static_cast<size_t>(a.experts);
  const size_t off_counts = 512;
  const size_t off_maps = (off_counts + sizeof(uint32_t) * a.experts + 127) / 128 * 128;
  const size_t meta_bytes = off_maps + map_bytes;
  const void* const staging_before = plan->staging.ptr;
  if (!plan->meta.reserve(meta_bytes) || !plan->staging.reserve(meta_bytes) ||
      !plan->worklist.reserve(sizeof(bmoe_tile) * static_cast<size_t>(tiles)) ||
      !plan->workspace.reserve(layout.bytes)) {
    return BMOE_CUDA_ERROR;
  }
  if (plan->setup_done == nullptr) {
    if (cudaEventCreateWithFlags(&plan->setup_done, cudaEventDisableTiming) != cudaSuccess) {
      return BMOE_CUDA_ERROR;
    }
  } else if (cudaEventSynchronize(plan->setup_done) != cudaSuccess) {
    // the previous set-up copy still reads the staging area
    return BMOE_CUDA_ERROR;
  }
  const bool staging_moved = plan->staging.ptr != staging_before;
  cudaStream_t stream = plan->setup_stream;
  uint8_t* const stage = static_cast<uint8_t*>(plan->staging.ptr);
  uint8_t* const meta = static_cast<uint8_t*>(plan->meta.ptr);

  // ---- queue and status words, counts, one TMA descriptor triple per active expert ----
  const uint32_t tail = policy.tail_tiles < tiles ? policy.tail_tiles : tiles;
  const uint32_t main_end = tiles - tail;
  std::memset(stage, 0, off_counts);
  reinterpret_cast<uint32_t*>(stage)[1] = main_end;  // tail counter starts after the main part
  if (!dev_counts) {
    std::memcpy(stage + off_counts, a.tokens_per_expert, sizeof(uint32_t) * a.experts);
  }
  CUtensorMap* const maps_a = reinterpret_cast<CUtensorMap*>(stage + off_maps);
  CUtensorMap* const maps_b = maps_a + a.experts;
  CUtensorMap* const maps_d = maps_b + a.experts;
  // B descriptors survive in the staging area from the previous initialize when the
  // layout of that area, the shape and the box are the same; only experts whose weight
  // pointer changed are encoded again.
  const uint32_t b_box = tile_n / cta_group;
  const bool b_cache_valid = !staging_moved && plan->b_key_experts == a.experts &&
                             plan->b_key_n == a.n && plan->b_key_k == a.k &&
                             plan->b_key_box == b_box && plan->b_key_type == a.data_type &&
                             plan->b_encoded_for.size() == a.experts;
  if (!b_cache_valid) plan->b_encoded_for.assign(a.experts, nullptr);
  plan->b_key_experts = a.experts;
  plan->b_key_n = a.n;
  plan->b_key_k = a.k;
  plan->b_key_box = b_box;
  plan->b_key_type = a.data_type;
  // Rows of the A box: 128, or fewer when no expert has that many rows (single-CTA tiles
  // only; see GemmParams::a_box_bytes).
  uint32_t a_box_rows = 128;
  if (cta_group == 1 && !dev_counts) {
    uint32_t most = 0;
    for (uint32_t e = 0; e < a.experts; ++e) {
      if (a.tokens_per_expert[e] > most) most = a.tokens_per_expert[e];
    }
    if (most < 128) a_box_rows = most < 8 ? 8u : (most + 7u) / 8u * 8u;
  }
  if (packed && !encode_matrix(&maps_a[0], a.packed_a, a.packed_rows, a.k, a_box_rows, operand)) {
    return BMOE_CUDA_ERROR;
  }
  for (uint32_t e = 0; e < a.experts; ++e) {
    const uint64_t rows = host_counts[e];
    if (rows == 0) {
      if (!packed || e != 0) std::memset(&maps_a[e], 0, sizeof(CUtensorMap));
      std::memset(&maps_b[e], 0, sizeof(CUtensorMap));
      std::memset(&maps_d[e], 0, sizeof(CUtensorMap));
      plan->b_encoded_for[e] = nullptr;
      continue;
    }
    if (!packed && !encode_matrix(&maps_a[e], a.a[e], rows, a.k, a_box_rows, operand)) {
      return BMOE_CUDA_ERROR;
    }
    if (plan->b_encoded_for[e] != a.b[e]) {
      if (!encode_matrix(&maps_b[e], a.b[e], a.n, a.k, b_box, operand)) return BMOE_CUDA_ERROR;
      plan->b_encoded_for[e] = a.b[e];
    }
    if (!pushed && !encode_matrix(&maps_d[e], a.d[e], rows, a.n, 32,
                                  out_f32 ? Elem::kF32 : Elem::kBf16)) {
      return BMOE_CUDA_ERROR;
    }
  }
  if (cudaMemcpyAsync(meta, stage, meta_bytes, cudaMemcpyHostToDevice, stream) != cudaSuccess) {
    return BMOE_CUDA_ERROR;
  }

  // ---- worklist built on the device from the device copy of the counts ----
  bmoe_worklist_request request;
  request.experts = a.experts;
  request.n = a.n;
  request.tile_m = tile_m;
  request.tile_n = tile_n;
  request.order = policy.order;
  request.raster = raster;
  int rc = bmoe_worklist_build(dev_counts ? a.tokens_per_expert_dev
                                          : reinterpret_cast<const uint32_t*>(meta + off_counts),
                               &request,
                               static_cast<bmoe_tile*>(plan->worklist.ptr), tiles,
                               plan->workspace.ptr, stream);
  if (rc != BMOE_OK) return rc;
  if (cudaEventRecord(plan->setup_done, stream) != cudaSuccess) return BMOE_CUDA_ERROR;

  // ---- launch parameters ----
  const CUtensorMap* const dev_maps = reinterpret_cast<const CUtensorMap*>(meta + off_maps);
  bmoe::GemmParams& p = plan->params;
  p = bmoe::GemmParams{};
  p.tmap_a = dev_maps;
  p.tmap_b = dev_maps + a.experts;
  p.tmap_d = dev_maps + 2 * static_cast<size_t>(a.experts);
  p.tiles = static_cast<const bmoe_tile*>(plan->worklist.ptr);
  p.tile_count = tiles;
  p.k_blocks = fp8 ? (a.k + 127) / 128 : (a.k + 63) / 64;   // 128 bytes of a row each
  p.fp8 = fp8 ? 1u : 0u;
  p.check_experts = a.experts;
  p.check_n = a.n;
  p.check_k_bytes = fp8 ? a.k : 2u * a.k;
  p.check_a_rows = packed ? a.packed_rows : 0;
  p.sched_mode = policy.sched_mode;
  p.claim_size = policy.claim_size;
  p.main_end = main_end;
  p.lookahead = policy.sched_mode == bmoe::kSchedStatic ? 0u : 1u;
  p.queue = reinterpret_cast<uint32_t*>(meta);
  p.status = reinterpret_cast<bmoe::DeviceStatus*>(
      meta + 256);
  p.tile_visits = nullptr;
  p.cta_tiles = nullptr;
  p.wait_budget_ns = 1000000000ull;  // 1 s per wait, then the kernel gives up
  p.a_box_bytes = a_box_rows * 128u;
  if (packed) {
    // first row of every expert in the packed buffer, as the worklist builder left it
    p.a_row_offsets = reinterpret_cast<const unsigned long long*>(
        static_cast<const uint8_t*>(plan->workspace.ptr) + layout.off_row_offsets);
  }
  plan->needs_push = pushed;
  if (dev_counts) {
    p.tile_count_dev = reinterpret_cast<const uint32_t*>(
        static_cast<const uint8_t*>(plan->workspace.ptr) + layout.off_totals +
        offsetof(bmoe_worklist_totals, total_tiles));
  }

  plan->tile_n = tile_n;
  plan->stats_n = a.n;
  plan->cta_group = cta_group;
  plan->out_f32 = out_f32;
  plan->units = policy.one_cta_per_tile ? tiles : (tiles < unit_budget ? tiles : unit_budget);
  if (dev_counts) plan->units = unit_budget;   // the tile total is not known here

  plan->stats.threadblock_count = plan->units * cta_group;
  plan->stats.workspace_bytes =
      plan->meta.bytes + plan->worklist.bytes + plan->workspace.bytes;
  plan->stats.total_tiles = tiles;
  plan->stats.tile_m = tile_m;
  plan->stats.tile_n = tile_n;
  plan->stats.resolved_scheduler = policy.scheduler;
  plan->stats.claim_size = policy.claim_size;
  plan->stats.hybrid_tail_tiles = tail;
  plan->stats.cta_group = cta_group;
  plan->stats.stages = bmoe::gemm_stage_count(tile_n, cta_group);
  plan->stats.dynamic_smem_bytes = bmoe::gemm_smem_bytes(tile_n, cta_group);
  plan->stats.launches = 0;
  plan->stats.sm_count = static_cast<uint32_t>(sm_count);
  plan->ready = true;
  return BMOE_OK;
}

int bmoe_preload_kernels(void) {
  cudaError_t rc = bmoe::preload_gemm_kernels();
  if (rc == cudaSuccess) rc = bmoe::preload_worklist_kernels();
  if (rc == cudaSuccess) rc = bmoe::preload_permute_kernels();
  if (rc == cudaSuccess) rc = bmoe::preload_exchange_kernels();
  if (rc == cudaSuccess) rc = bmoe::preload_probe_kernels();
  return rc == cudaSuccess ? BMOE_OK : BMOE_CUDA_ERROR;
}

int bmoe_plan_set_gate(bmoe_plan* plan, const uint32_t* flags_dev, uint32_t epoch,
                       uint32_t ranks, uint32_t self, const uint8_t* group_of_expert_dev) {
  if (plan == nullptr || !plan->ready) return BMOE_INVALID_ARGUMENT;
  bmoe::GemmParams& p = plan->params;
  p.gate_copy_mask = nullptr;
  p.gate_copy_plane = 0;
  p.expand_records = nullptr;
  if (flags_dev == nullptr || ranks <= 1) {
    p.gate_flags = nullptr;
    p.gate_group_of = nullptr;
    return BMOE_OK;
  }
  if (self >= ranks || ranks > 32 || group_of_expert_dev == nullptr) return BMOE_INVALID_ARGUMENT;
  p.gate_flags = flags_dev;
  p.gate_group_of = group_of_expert_dev;
  p.gate_epoch = epoch;
  p.gate_ranks = ranks;
  p.gate_self = self;
  return BMOE_OK;
}

int bmoe_plan_set_gate_copies(bmoe_plan* plan, const uint32_t* copy_mask_dev) {
  if (plan == nullptr || !plan->ready) return BMOE_INVALID_ARGUMENT;
  bmoe::GemmParams& p = plan->params;
  if (copy_mask_dev != nullptr && p.gate_flags == nullptr) return BMOE_INVALID_ARGUMENT;
  p.gate_copy_mask = copy_mask_dev;
  p.gate_copy_plane = copy_mask_dev != nullptr ? BMOE_EP_COPY_FLAGS(p.gate_ranks) : 0u;
  return BMOE_OK;
}

int bmoe_plan_set_expand(bmoe_plan* plan, const void* records_dev, const uint32_t* counts_dev,
                         uint32_t* next_dev, uint32_t* done_dev, void* a_dev,
                         uint64_t rows_cap, uint32_t row_bytes, uint32_t record_cap,
                         uint32_t groups) {
  if (plan == nullptr || !plan->ready) return BMOE_INVALID_ARGUMENT;
  bmoe::GemmParams& p = plan->params;
  if (records_dev == nullptr) {
    p.expand_records = nullptr;
    return BMOE_OK;
  }
  if (p.gate_flags == nullptr || counts_dev == nullptr || next_dev == nullptr ||
      done_dev == nullptr || a_dev == nullptr || rows_cap == 0 || row_bytes == 0 ||
      row_bytes % 16 != 0 || record_cap == 0 || groups == 0 || groups > BMOE_EP_MAX_GROUPS ||
      misaligned16(a_dev)) {
    return BMOE_INVALID_ARGUMENT;
  }
  p.expand_records = static_cast<const uint2*>(records_dev);
  p.expand_count = counts_dev;
  p.expand_next = next_dev;
  p.expand_done = done_dev;
  p.expand_a = static_cast<uint4*>(a_dev);
  p.expand_rows_cap = rows_cap;
  p.expand_vec_per_row = row_bytes / 16;
  p.expand_cap = record_cap;
  p.expand_groups = groups;
  return BMOE_OK;
}

int bmoe_plan_set_push(bmoe_plan* plan, const void* origin_dev,
                       const uint32_t* expert_row_dev, void* const* y_bases_dev,
                       uint32_t ranks, uint64_t y_rows_cap) {
  if (plan == nullptr || !plan->ready) return BMOE_INVALID_ARGUMENT;
  bmoe::GemmParams& p = plan->params;
  if (origin_dev == nullptr) {
    p.push_origin = nullptr;
    return BMOE_OK;
  }
  if (plan->out_f32 || expert_row_dev == nullptr || y_bases_dev == nullptr || ranks == 0 ||
      y_rows_cap == 0) {
    return BMOE_INVALID_ARGUMENT;
  }
  p.push_origin = static_cast<const long long*>(origin_dev);
  p.push_expert_row = expert_row_dev;
  p.push_bases = reinterpret_cast<uint4* const*>(y_bases_dev);
  p.push_rows_cap = y_rows_cap;
  p.push_vec_per_row = plan->stats_n / 8;
  p.push_ranks = ranks;
  return BMOE_OK;
}

int bmoe_plan_run(bmoe_plan* plan, void* stream) {
  if (plan == nullptr || !plan->ready) return BMOE_INVALID_ARGUMENT;
  if (plan->stats.active_experts == 0) return BMOE_OK;
  if (plan->needs_push && plan->params.push_origin == nullptr) return BMOE_INVALID_ARGUMENT;
  cudaStream_t s = stream == nullptr ? plan->default_stream
                                     : static_cast<cudaStream_t>(stream);
  if (s != plan->setup_stream &&
      cudaStreamWaitEvent(s, plan->setup_done, 0) != cudaSuccess) {
    return BMOE_CUDA_ERROR;
  }
  const cudaError_t err =
      bmoe::launch_grouped_gemm(plan->params, plan->tile_n, plan->cta_group, plan->out_f32,
                                plan->units, s);
  plan->last_stream = s;
  if (err != cudaSuccess) return BMOE_CUDA_ERROR;
  plan->stats.launches += 1;
  return BMOE_OK;
}

int bmoe_plan_stats_get(const bmoe_plan* plan, bmoe_plan_stats* out) {
  if (out == nullptr) return BMOE_INVALID_ARGUMENT;
  *out = plan == nullptr ? bmoe_plan_stats{} : plan->stats;
  return BMOE_OK;
}

int bmoe_plan_poll(bmoe_plan* plan, bmoe_device_report* report) {
  if (plan == nullptr || !plan->ready) return BMOE_INVALID_ARGUMENT;
  if (report != nullptr) std::memset(report, 0, sizeof(*report));
  if (plan->stats.active_experts == 0) return BMOE_OK;
  if (cudaStreamSynchronize(plan->last_stream) != cudaSuccess) return BMOE_CUDA_ERROR;
  bmoe::DeviceStatus st{};
  if (cudaMemcpy(&st, plan->params.status, sizeof(st), cudaMemcpyDeviceToHost) !=
      cudaSuccess) {
    return BMOE_CUDA_ERROR;
  }
  if (st.count == 0) return BMOE_OK;
  if (report != nullptr) {
    report->code = st.code;
    report->cta = st.cta;
    report->role = st.role;
    report->tile = st.tile;
    report->stage = st.stage;
    report->aux = st.aux;
    report->count = st.count;
  }
  // Rearm the status record and the queue so the plan stays usable.
  uint32_t control_init[128];
  std::memset(control_init, 0, sizeof(control_init));
  control_init[1] = plan->params.main_end;
  cudaMemcpy(plan->meta.ptr, control_init, sizeof(control_init), cudaMemcpyHostToDevice);
  return BMOE_DEVICE_TIMEOUT;
}

int bmoe_plan_read_worklist(bmoe_plan* plan, bmoe_tile* tiles_host, uint32_t capacity,
                            uint32_t* count_out) {
  if (plan == nullptr || !plan->ready) return BMOE_INVALID_ARGUMENT;
  const uint32_t total = plan->stats.total_tiles;
  if (count_out != nullptr) *count_out = total;
  const uint32_t n_copy = capacity < total ? capacity : total;
  if (n_copy == 0) return BMOE_OK;
  if (tiles_host == nullptr) return BMOE_INVALID_ARGUMENT;
  if (cudaStreamSynchronize(plan->setup_stream) != cudaSuccess) return BMOE_CUDA_ERROR;
  return cudaMemcpy(tiles_host, plan->worklist.ptr, sizeof(bmoe_tile) * n_copy,
                    cudaMemcpyDeviceToHost) == cudaSuccess
             ? BMOE_OK
             : BMOE_CUDA_ERROR;
}

int bmoe_plan_set_observers(bmoe_plan* plan, uint32_t* tile_visits_dev,
                            uint32_t* cta_tiles_dev) {
  if (plan == nullptr || !plan->ready) return BMOE_INVALID_ARGUMENT;
  plan->params.tile_visits = tile_visits_dev;
  plan->params.cta_tiles = cta_tiles_dev;
  return BMOE_OK;
}

int bmoe_plan_set_trace(bmoe_plan* plan, uint64_t* trace_dev) {
  if (plan == nullptr || !plan->ready) return BMOE_INVALID_ARGUMENT;
  plan->params.trace = trace_dev;
  return BMOE_OK;
}

int bmoe_grouped_gemm(const bmoe_gemm_args* args) {
  if (args == nullptr) return BMOE_INVALID_ARGUMENT;
  bmoe_plan* plan = bmoe_plan_create();
  if (plan == nullptr) return BMOE_CUDA_ERROR;
  int rc = bmoe_plan_initialize(plan, args);
  if (rc == BMOE_OK) rc = bmoe_plan_run(plan, args->stream);
  // The plan owns the worklist and descriptors the kernel reads: wait for the
  // launch before releasing them.
  if (rc == BMOE_OK) rc = bmoe_plan_poll(plan, nullptr);
  bmoe_plan_destroy(plan);
  return rc;
}

const char* bmoe_build_info(void) {
  return "bmoe_b200: sm_100a, tcgen05/TMEM/TMA grouped GEMM, CUDA runtime "
#define BMOE_STR2(x) #x
#define BMOE_STR(x) BMOE_STR2(x)
         BMOE_STR(CUDART_VERSION);
}

}  // extern "C"
