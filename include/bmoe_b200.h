/*
 * bmoe_b200.h - C interface of the B200 (sm_100a) MoE grouped-GEMM engine.
 *
 * Plain C: pointers, sizes and integer status codes only. Every entry point
 * names the reference interface it stands in for (paths are relative to the
 * reference project root). The C++ classes in include/blackwell_moe/ are thin
 * wrappers over these functions and live in the same shared library.
 *
 * Conventions
 *   - "dev" pointers are CUDA device pointers, "host" pointers are host memory.
 *   - stream arguments are cudaStream_t values passed as void* (NULL = default).
 *   - All functions return a bmoe_status value unless stated otherwise and
 *     never throw.
 *   - There is no CPU implementation behind the device entry points: without a
 *     compute-capability-10.0 GPU they return BMOE_UNSUPPORTED_DEVICE or
 *     BMOE_CUDA_ERROR.
 */
#ifndef BMOE_B200_H_
#define BMOE_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------------ */
/* Status codes. Values 0-6 are the ordinals of blackwell_moe::KernelStatus  */
/* (include/blackwell_moe/kernels/grouped_gemm.cuh:30-38); 7 is appended.    */
/* ------------------------------------------------------------------------ */
enum bmoe_status {
  BMOE_OK = 0,
  BMOE_INVALID_ARGUMENT = 1,
  BMOE_UNSUPPORTED_DATA_TYPE = 2,
  BMOE_UNSUPPORTED_SCHEDULER = 3,
  BMOE_UNSUPPORTED_DEVICE = 4,
  BMOE_CUDA_ERROR = 5,
  BMOE_BACKEND_ERROR = 6, /* reference "CUTLASS error" slot; never returned */
  BMOE_DEVICE_TIMEOUT = 7 /* a bounded in-kernel wait expired */
};

/* Replaces kernel_status_string (grouped_gemm.cuh:40; defined only in
 * baselines/cutlass/cutlass_baseline.cu:165-176 in the reference). */
const char* bmoe_status_string(int status);

/* Scheduling policies: ordinals of blackwell_moe::SchedulerKind
 * (include/blackwell_moe/scheduler/scheduler.cuh:12-18) plus CLC. */
enum bmoe_scheduler {
  BMOE_SCHED_EXPERT_ORDER = 0,
  BMOE_SCHED_STATIC_PERSISTENT = 1, /* a.k.a. sorted_static */
  BMOE_SCHED_DYNAMIC_QUEUE = 2,
  BMOE_SCHED_COMPACTED = 3,
  BMOE_SCHED_AUTO = 4,
  BMOE_SCHED_CLC = 5
};

/* The 20-byte worklist record, byte-identical to blackwell_moe::ExpertTile
 * (include/blackwell_moe/work_tile.cuh:13-21). */
typedef struct bmoe_tile {
  uint32_t expert_id;
  uint32_t tile_m;
  uint32_t tile_n;
  uint32_t valid_m;
  uint32_t valid_n;
} bmoe_tile;

/* ======================================================================== */
/* 1. Host model: workload generator, worklist, policies, metrics, dispatch  */
/* ======================================================================== */

/* blackwell_moe::WorkloadConfig (include/blackwell_moe/problem.hpp:16-25).
 * distribution: 0 uniform, 1 heavy_hitter, 2 sparse, 3 zipf, 4 heavy_sparse
 * (appended: hot set in front, idle set at the back; no reference counterpart). */
typedef struct bmoe_workload_config {
  uint32_t experts;
  uint32_t distribution;
  uint64_t total_tokens;
  uint64_t seed;
  double zipf_alpha;
  double heavy_hitter_fraction;
  double heavy_hitter_token_share;
  double inactive_expert_fraction;
} bmoe_workload_config;

/* Replaces generate_workload (src/workload/workload.cpp:100-113).
 * counts_out: host array [experts]. Invalid configs -> BMOE_INVALID_ARGUMENT. */
int bmoe_generate_workload(const bmoe_workload_config* config,
                           uint32_t* counts_out);

/* blackwell_moe::WorkloadMetrics (include/blackwell_moe/workload.hpp:10-19). */
typedef struct bmoe_workload_metrics {
  double mean_tokens;
  double coefficient_of_variation;
  double max_over_mean;
  double inactive_expert_ratio;
  double small_m_expert_ratio;
  double tile_count_cv;
  uint32_t active_experts;
  uint32_t reserved;
  uint64_t total_tiles;
} bmoe_workload_metrics;

/* Replaces compute_workload_metrics (src/workload/workload.cpp:127-172). */
int bmoe_workload_metrics_compute(const uint32_t* counts, uint32_t experts,
                                  uint32_t n, uint32_t tile_m, uint32_t tile_n,
                                  bmoe_workload_metrics* out);

/* Worklist orders. */
enum bmoe_worklist_order {
  BMOE_ORDER_EXPERT = 0,       /* build_expert_tiles order */
  BMOE_ORDER_SORTED_BY_WORK = 1 /* order_by_descending_expert_tiles order */
};
/* Traversal inside one expert's tile grid. */
enum bmoe_raster {
  BMOE_RASTER_N_FASTEST = 0, /* reference order: tile_m outer, tile_n inner */
  BMOE_RASTER_M_FASTEST = 1  /* tile_n outer, tile_m inner (L2-friendly) */
};

/* Number of tiles build_expert_tiles would emit. Returns UINT64_MAX when a
 * tile dimension is zero. */
uint64_t bmoe_host_tile_count(const uint32_t* counts, uint32_t experts,
                              uint32_t n, uint32_t tile_m, uint32_t tile_n);

/* Replaces build_expert_tiles / order_by_descending_expert_tiles
 * (src/scheduler/scheduler.cpp:37-60, 80-103) on the host. Writes at most
 * `capacity` records and always reports the full count in *count_out. */
int bmoe_host_build_tiles(const uint32_t* counts, uint32_t experts, uint32_t n,
                          uint32_t tile_m, uint32_t tile_n, uint32_t order,
                          uint32_t raster, bmoe_tile* tiles_out,
                          uint64_t capacity, uint64_t* count_out);

/* blackwell_moe::ScheduleMetrics (scheduler.cuh:26-39). */
typedef struct bmoe_schedule_metrics {
  uint64_t total_tiles;
  uint64_t total_valid_elements;
  uint64_t total_padded_elements;
  uint64_t expert_switches;
  uint64_t min_tiles_per_cta;
  uint64_t max_tiles_per_cta;
  double mean_cta_work;
  double max_cta_work;
  double cta_work_cv;
  double tail_ratio;
  double estimated_utilization;
  double useful_work_ratio;
} bmoe_schedule_metrics;

/* Replaces simulate_scheduler + compute_schedule_metrics
 * (src/scheduler/scheduler.cpp:124-211). tiles_out receives the per-CTA tile
 * lists back to back (capacity records), cta_offsets_out[cta_count + 1] their
 * boundaries; either may be NULL. cta_count == 0 -> BMOE_INVALID_ARGUMENT. */
int bmoe_host_simulate(uint32_t scheduler, const uint32_t* counts,
                       uint32_t experts, uint32_t n, uint32_t tile_m,
                       uint32_t tile_n, uint32_t cta_count,
                       bmoe_tile* tiles_out, uint64_t capacity,
                       uint64_t* cta_offsets_out,
                       bmoe_schedule_metrics* metrics_out);

/* RoutingFeatures (python/blackwell_moe_tirx/dispatch.py:16-27). */
typedef struct bmoe_routing_features {
  double mean_m;
  double cv_m;
  double max_over_mean_m;
  double inactive_expert_ratio;
  double small_m_expert_ratio;
  double expert_tile_cv;
  double max_expert_tiles_over_mean;
  uint64_t active_tiles;
  double tiles_per_cta;
  double useful_work_ratio;
} bmoe_routing_features;

/* Replaces routing_features (dispatch.py:42-83). */
int bmoe_routing_features_compute(const uint32_t* counts, uint32_t experts,
                                  uint32_t n, uint32_t tile_m, uint32_t tile_n,
                                  uint32_t cta_count,
                                  bmoe_routing_features* out);

/* Launch variants, in the order of KERNEL_VERSIONS minus v0_5
 * (python/blackwell_moe_tirx/kernels/registry.py:45-106). */
enum bmoe_variant {
  BMOE_VARIANT_NONPERSISTENT = 0,
  BMOE_VARIANT_STATIC_WS = 1,
  BMOE_VARIANT_DYNAMIC_CLAIM1 = 2,
  BMOE_VARIANT_CHUNKED = 3,
  BMOE_VARIANT_HYBRID = 4,
  BMOE_VARIANT_CLC = 5
};

/* Replaces select_kernel with the default DispatchThresholds
 * (dispatch.py:30-39, 86-114). thresholds may be NULL (defaults) or point to
 * six doubles in the field order of DispatchThresholds. */
int bmoe_select_variant(const bmoe_routing_features* features,
                        const double* thresholds, uint32_t* variant_out);
const char* bmoe_variant_name(uint32_t variant);

/* The engine's own rule, the one a plan applies for BMOE_SCHED_AUTO (fitted on B200
 * measurements of this engine; the reference never picks launch control,
 * dispatch.py:93-94, and its bootstrap values are explicitly provisional,
 * agent/evaluation_contract.md:41-48): one CTA per tile when no unit gets more than one
 * tile, the static stride when the active experts hold `weight_stream_mean_rows` rows or
 * fewer on average (a pure weight stream of equal-cost tiles), launch control otherwise.
 * rule may be NULL (fitted values) or point to two doubles
 * {nonpersistent_tiles_per_cta, weight_stream_mean_rows}. */
int bmoe_select_variant_fitted(const bmoe_routing_features* features, const double* rule,
                               uint32_t* variant_out);

/* ======================================================================== */
/* 2. Device worklist builder                                                */
/* ======================================================================== */

/* Totals written by the builder (device memory, 32 bytes). */
typedef struct bmoe_worklist_totals {
  uint32_t total_tiles;
  uint32_t active_experts;
  uint64_t total_rows;           /* sum of counts */
  uint64_t total_valid_elements; /* sum of counts * n */
  uint32_t overflow;             /* 1 if total_tiles exceeded tile_capacity or 2^32 */
  uint32_t reserved;
} bmoe_worklist_totals;

/* Byte offsets of the arrays inside the builder workspace for `experts`. */
typedef struct bmoe_worklist_layout {
  size_t bytes;                   /* workspace size */
  size_t off_totals;              /* bmoe_worklist_totals */
  size_t off_row_offsets;         /* uint64 [experts + 1] exclusive prefix of counts */
  size_t off_expert_m_tiles;      /* uint32 [experts] ceil(count / tile_m) */
  size_t off_expert_tiles;        /* uint32 [experts] m_tiles * n_tiles */
  size_t off_tile_offsets;        /* uint32 [experts + 1] prefix of expert_tiles by id */
  size_t off_active_ids;          /* uint32 [experts] ascending ids of experts with
                                     tokens, padded with 0xFFFFFFFF */
  size_t off_visit_order;         /* uint32 [experts] expert visited at position p */
  size_t off_visit_tile_offsets;  /* uint32 [experts + 1] prefix of tiles in visit order */
} bmoe_worklist_layout;

int bmoe_worklist_layout_for(uint32_t experts, bmoe_worklist_layout* out);

/* Largest expert count the single-CTA planning kernel accepts. */
#define BMOE_WORKLIST_MAX_EXPERTS 16384u
/* Largest expert count for BMOE_ORDER_SORTED_BY_WORK (the stable descending sort is a
 * rank computation, experts^2 / 1024 steps per thread; 4096 experts take about 50 us). */
#define BMOE_WORKLIST_MAX_SORTED_EXPERTS 4096u

typedef struct bmoe_worklist_request {
  uint32_t experts;
  uint32_t n;
  uint32_t tile_m;
  uint32_t tile_n;
  uint32_t order;  /* bmoe_worklist_order */
  uint32_t raster; /* bmoe_raster */
} bmoe_worklist_request;

/* On-device statement of build_expert_tiles /
 * order_by_descending_expert_tiles (src/scheduler/scheduler.cpp:37-60, 80-103)
 * and of the active-expert filter of the reference plan
 * (baselines/cutlass/cutlass_baseline.cu:243-266): two integer kernels,
 * enqueued on `stream`, no host synchronisation.
 *   counts_dev    uint32 [experts]
 *   tiles_dev     bmoe_tile [tile_capacity]; records beyond capacity are
 *                 dropped and totals.overflow is set
 *   workspace_dev bmoe_worklist_layout_for(experts).bytes bytes, 256-aligned */
int bmoe_worklist_build(const uint32_t* counts_dev,
                        const bmoe_worklist_request* request,
                        bmoe_tile* tiles_dev, uint32_t tile_capacity,
                        void* workspace_dev, void* stream);

/* Largest expert count bmoe_worklist_build_static accepts. */
#define BMOE_WORKLIST_STATIC_MAX_EXPERTS 1024u

/* Allocation-free variant of bmoe_worklist_build. It has no counterpart in the
 * reference. It exists for callers that must not allocate device memory at the
 * point where routing counts become known: code running inside a serving loop
 * whose memory pool is fixed up front, a plug-in that is handed buffers by its
 * host framework and is forbidden from calling cudaMalloc (which also
 * synchronises the device), or a caller that has already handed all free
 * memory to another allocator. The builder's auxiliary arrays (prefix sums,
 * active-expert list, visiting order) live in a fixed array inside the library
 * image instead of a caller-provided workspace; the caller passes only the
 * inputs and the outputs:
 *   counts_dev       uint32 [experts]                       (input)
 *   tiles_dev        bmoe_tile [tile_capacity]              (output)
 *   totals_out_dev   one bmoe_worklist_totals, may be NULL  (output)
 * Limits and rules:
 *   - request->experts <= BMOE_WORKLIST_STATIC_MAX_EXPERTS, otherwise
 *     BMOE_INVALID_ARGUMENT is returned and nothing is launched. The array
 *     costs about 34 KB of device memory on every GPU that loads the library,
 *     for the life of the process.
 *   - No cudaMalloc / cudaFree or other allocating call is made.
 *   - The first call on each device looks up the device address of the array
 *     (cudaGetSymbolAddress); make that first call outside any stream capture.
 *     bmoe_preload_kernels() performs the same lookup, so a caller that preloads
 *     has already met this rule. The lookup result is cached per device ordinal
 *     for the life of the process (two host threads making their first call
 *     together both store the same address); after cudaDeviceReset the cache
 *     is stale and the entry point must not be used again in that process.
 *   - All calls on one device share the array. Every word a call reads from it
 *     is written by that call first, so stale contents from an earlier call
 *     are harmless, but two calls whose kernels overlap on the GPU (different
 *     streams, no ordering between them) race and give undefined results. */
int bmoe_worklist_build_static(const uint32_t* counts_dev,
                               const bmoe_worklist_request* request,
                               bmoe_tile* tiles_dev, uint32_t tile_capacity,
                               bmoe_worklist_totals* totals_out_dev,
                               void* stream);

/* ======================================================================== */
/* 3. Grouped-GEMM plan                                                      */
/* ======================================================================== */

/* blackwell_moe::GroupedGemmArguments (grouped_gemm.cuh:12-28) followed by the
 * engine extensions; zero (raster: negative) selects the engine default. */
typedef struct bmoe_gemm_args {
  const void* const* a;              /* host array [experts] of device pointers */
  const void* const* b;
  void* const* d;
  const uint32_t* tokens_per_expert; /* host array [experts] */
  uint32_t experts;
  uint32_t n;
  uint32_t k;
  uint32_t data_type; /* 0 = BF16; 1 = FP8 E4M3: a[] and b[] hold one byte per element
                         (no scales), FP32 accumulation, D as for BF16; k must then be a
                         multiple of 16. The reference declares the type and rejects it
                         (grouped_gemm.cuh:10, cutlass_baseline.cu:211-213); so do the
                         C++ Bf16GroupedGemmPlan and the one-shot launcher. Other values:
                         BMOE_UNSUPPORTED_DATA_TYPE. */
  uint32_t scheduler; /* bmoe_scheduler */
  uint32_t claim_size;
  uint32_t hybrid_tail_tiles;
  uint32_t cta_count;
  uint32_t tile_n;    /* 64, 128 or 256 output columns per tile; 0 = 256, or 128 when the
                         problem is a single wave either way (single-CTA tiles) */
  uint32_t cta_group; /* 1 = 128-row tiles, 2 = CTA pairs computing 256 x 256 tiles,
                         0 = chosen from the routing (pairs unless they pad > 10 % more) */
  int32_t raster_along_m;
  uint32_t output_f32; /* 0: D is BF16 (reference contract); 1: D is row-major FP32,
                          the unrounded accumulators (direct_cute_gemm.cuh:16-18) */
  void* stream;
  /* Packed layout (appended; zero = the pointer-array form above). When packed_a is
   * set, the rows of all experts lie back to back in ONE row-major buffer
   * [packed_rows, k] in expert order (row offsets = exclusive prefix sum of the
   * counts, derived on the device); a[] is then ignored and one tensor map serves every
   * expert, so a re-plan with new counts encodes no per-expert A descriptor. B
   * descriptors of experts whose pointer did not change since the plan's previous
   * initialize are reused as well. */
  const void* packed_a;
  uint64_t packed_rows;
  /* 1: D is never stored through the plan (results leave through bmoe_plan_set_push,
   * which must then be set before run); d[] is ignored and no D descriptor is made. */
  uint32_t results_pushed;
  uint32_t reserved0;
  /* Counts that only exist on the device (appended; NULL = the host array above). When
   * set, uint32 [experts] in device memory holds the rows per expert, written by work
   * that precedes initialize in `stream`; the host never reads it, so a step needs no
   * host synchronisation between routing and the GEMM launch. The worklist is built from
   * it on the device, the kernel reads the tile total from device memory and the grid is
   * the full persistent grid. Requires packed_a (packed_rows = row capacity of the
   * buffer, an upper bound of the routed rows), results_pushed = 1, cta_group 1 or 2
   * (0 = 2 when n > 128), tile_n 0 (= 256) or explicit, a persistent policy
   * (expert_order, static_persistent, compacted, dynamic_queue; no hybrid tail).
   * tokens_per_expert is then ignored; stats report capacities. */
  const uint32_t* tokens_per_expert_dev;
} bmoe_gemm_args;

/* blackwell_moe::GroupedGemmPlanStats (grouped_gemm.cuh:42-46) + extensions. */
typedef struct bmoe_plan_stats {
  uint32_t active_experts;
  uint32_t threadblock_count;
  uint64_t workspace_bytes;
  uint32_t total_tiles;
  uint32_t tile_m;
  uint32_t tile_n;
  uint32_t resolved_scheduler;
  uint32_t claim_size;
  uint32_t hybrid_tail_tiles;
  uint32_t cta_group;
  uint32_t stages;
  uint32_t dynamic_smem_bytes;
  uint32_t launches; /* kernel launches enqueued by run() since initialize */
  uint32_t sm_count; /* multiprocessors of the plan's device */
} bmoe_plan_stats;

/* What a kernel recorded when it gave up on a bounded wait. */
typedef struct bmoe_device_report {
  uint32_t code;  /* 0 = clean; otherwise a BMOE_DEV_* site code */
  uint32_t cta;
  uint32_t role;  /* 0 scheduler, 1 producer, 2 mma, 3 epilogue */
  uint32_t tile;
  uint32_t stage;
  uint32_t aux;
  uint32_t count; /* CTAs that reported */
  uint32_t reserved;
} bmoe_device_report;

typedef struct bmoe_plan bmoe_plan;

/* Replace Bf16GroupedGemmPlan's constructor / destructor / initialize / run /
 * stats (grouped_gemm.cuh:51-69; behaviour of
 * baselines/cutlass/cutlass_baseline.cu:179-377). */
bmoe_plan* bmoe_plan_create(void);
void bmoe_plan_destroy(bmoe_plan* plan);
int bmoe_plan_initialize(bmoe_plan* plan, const bmoe_gemm_args* args);
int bmoe_plan_run(bmoe_plan* plan, void* stream);
int bmoe_plan_stats_get(const bmoe_plan* plan, bmoe_plan_stats* out);

/* Synchronises the stream last used by run() and returns BMOE_DEVICE_TIMEOUT
 * (filling *report when non-NULL) if a kernel abandoned a wait. */
int bmoe_plan_poll(bmoe_plan* plan, bmoe_device_report* report);

/* Copies the plan's device worklist back to the host (synchronises). */
int bmoe_plan_read_worklist(bmoe_plan* plan, bmoe_tile* tiles_host,
                            uint32_t capacity, uint32_t* count_out);

/* Optional device counters for exact-once checks (NULL disables):
 *   tile_visits_dev   uint32 [total_tiles], +1 by the CTA that ran the tile
 *   cta_tiles_dev     uint32 [threadblock_count], tiles run per scheduling unit
 *                     (CTA, or CTA pair when cta_group is 2: then only the first
 *                     threadblock_count / 2 entries are written)
 * The caller zeroes them. Mirrors the probe observables
 * (include/blackwell_moe/scheduler/scheduler_probe.cuh:24-28). */
int bmoe_plan_set_observers(bmoe_plan* plan, uint32_t* tile_visits_dev,
                            uint32_t* cta_tiles_dev);

/* Optional wait accounting (NULL disables): trace_dev is uint64
 * [threadblock_count][16]; per CTA, SM cycles spent blocked per role:
 *   [0] producer/tile info  [1] producer/free stage   [2] MMA/tile info
 *   [3] MMA/drained accumulator  [4] MMA/operand bytes [5] epilogue/tile info
 *   [6] epilogue/finished accumulator  [7] epilogue draining
 *   [8] tiles run  [9] kernel cycles  [10] MMA lane issuing. The caller zeroes it. No reference
 * counterpart (the reference measures with ncu only, tools/profile_ncu.sh). */
int bmoe_plan_set_trace(bmoe_plan* plan, uint64_t* trace_dev);

/* Replaces launch_grouped_gemm_baseline (grouped_gemm.cuh:71). */
int bmoe_grouped_gemm(const bmoe_gemm_args* args);

/* ======================================================================== */
/* 4. Scheduler probe                                                        */
/* ======================================================================== */

/* blackwell_moe::SchedulerProbeArguments (scheduler_probe.cuh:18-30). */
typedef struct bmoe_probe_args {
  const bmoe_tile* tiles;
  uint32_t tile_count;
  uint32_t cta_count;
  uint32_t claim_size;
  uint32_t work_scale;
  uint32_t* next_tile;
  uint32_t* tile_visits;
  uint64_t* tile_checksums;
  uint32_t* cta_tile_counts;
  uint64_t* cta_valid_elements;
  void* stream;
} bmoe_probe_args;

/* Replaces launch_scheduler_probe / device_scheduler_name
 * (src/kernels/scheduler_probe.cu:105-141). scheduler: 0 static, 1 queue. */
int bmoe_probe_launch(uint32_t scheduler, const bmoe_probe_args* args);
const char* bmoe_probe_scheduler_name(uint32_t scheduler);

/* ======================================================================== */
/* 5. Expert-parallel helpers (no counterpart in the reference, which has no  */
/*    multi-GPU code: agent/search_space.yaml:10-13)                          */
/* ======================================================================== */

/* Expert -> rank placement by tile-count balance. global_counts: host
 * uint32 [experts], summed over all ranks. Experts are taken in (more tiles
 * first, lower id first) order and given to the rank with the fewest tiles so
 * far (lowest rank on ties). max_experts_per_rank == 0 means no cap.
 * owner_out: host uint32 [experts]; rank_tiles_out: host uint64 [ranks] or NULL. */
int bmoe_ep_place_experts(const uint32_t* global_counts, uint32_t experts,
                          uint32_t ranks, uint32_t n, uint32_t tile_m,
                          uint32_t tile_n, uint32_t max_experts_per_rank,
                          uint32_t* owner_out, uint64_t* rank_tiles_out);

/* Row gather on the device: dst[i, :] = src[index[i], :], rows of row_bytes
 * bytes (a multiple of 16; both bases 16-byte aligned). index_dev: int64
 * [rows]; entries outside [0, src_rows) leave the destination row untouched.
 * The token permutation either side of the grouped GEMM (dispatch order,
 * expert-major packing, and their inverses). */
int bmoe_gather_rows(const void* src_dev, void* dst_dev, const int64_t* index_dev,
                     uint64_t rows, uint64_t src_rows, uint32_t row_bytes,
                     void* stream);

/* Row routing over peer memory (NVLink): for i in [0, rows)
 *   dst_bases[dst_rank[i]] + dst_row[i] * row_bytes  <-
 *   src_bases[src_rank[i]] + src_row[i] * row_bytes
 * src_bases_dev / dst_bases_dev: DEVICE arrays of n_src / n_dst base pointers
 * (own buffers or buffers of other GPUs opened with bmoe_peer_open). A NULL rank
 * array means entry 0 for every row, a NULL row array means row i. Rows whose
 * rank or row index is out of range (>= n_*, >= *_rows_cap) are skipped. One
 * kernel of plain loads and stores; max_ctas bounds its grid (0 = default) so it
 * can run beside another kernel. The expert-parallel dispatch (push token rows
 * into the owner's expert-major A) and combine (pull result rows back) are each
 * one call. row_bytes must be a multiple of 16. */
int bmoe_route_rows(const void* const* src_bases_dev, uint32_t n_src,
                    uint64_t src_rows_cap, const int32_t* src_rank_dev,
                    const int64_t* src_row_dev, void* const* dst_bases_dev,
                    uint32_t n_dst, uint64_t dst_rows_cap,
                    const int32_t* dst_rank_dev, const int64_t* dst_row_dev,
                    uint64_t rows, uint32_t row_bytes, uint32_t max_ctas,
                    void* stream);

/* Weighted top-k combine, the un-permute after the expert GEMMs: for t in [0, tokens)
 *   out[t, :] = bf16( sum_{j < top_k} w[t*top_k+j] *
 *                     float(src_bases[rank[t*top_k+j]][row[t*top_k+j], :]) )
 * FP32 accumulation, one fused multiply-add per term in ascending j, one BF16
 * rounding (nearest even) at the end. A NULL weight array means 1.0 for every
 * term, a NULL rank array means src_bases[0]. A negative row marks a dropped
 * assignment; it and any out-of-range rank / row contribute nothing. The source
 * buffers may belong to other GPUs (bmoe_peer_open), which makes this one kernel
 * the expert-parallel combine exchange and the reduction together. n must be a
 * multiple of 8. The reference leaves this step to its caller
 * (agent/search_space.yaml:13 treats the permutation as engine input). */
int bmoe_combine_topk(const void* const* src_bases_dev, uint32_t n_src,
                      uint64_t src_rows_cap, const int32_t* src_rank_dev,
                      const int64_t* src_row_dev, const float* weights_dev,
                      uint64_t tokens, uint32_t top_k, uint32_t n, void* out_dev,
                      uint32_t max_ctas, void* stream);

/* ---- Expert-parallel exchange overlapped with the grouped GEMM (peer memory) ----
 * No counterpart in the reference, which has no multi-GPU path; these are the data
 * movers either side of its grouped-GEMM interface for the expert-parallel
 * configuration. One rank per GPU; every pointer table below is a DEVICE array of
 * `ranks` base pointers (own buffer or bmoe_peer_open mappings).
 *
 * Flag arrays: every rank owns a zero-initialised uint32 array of
 * (BMOE_EP_MAX_GROUPS + 1) * ranks slots that all ranks map. Slot g*ranks + s holds
 * the last step ("epoch", increasing by one per step) for which source rank s has
 * delivered all of its rows of expert group g; slot BMOE_EP_MAX_GROUPS*ranks + s
 * the last step whose results rank s has returned. A rank never raises flags in
 * its own array. */
#define BMOE_EP_MAX_GROUPS 16u
#define BMOE_EP_LOCAL 0u   /* only rows whose owner is this rank; raises no flag */
#define BMOE_EP_REMOTE 1u  /* only rows owned by other ranks; raises the group flags */
#define BMOE_EP_ALL 2u
#define BMOE_EP_PACK 3u    /* only the rows of copy-engine blocks, into the local staging buffer */
/* Second flag plane, for rows that arrive as peer copies: slot
 * BMOE_EP_COPY_FLAGS(ranks) + g*ranks + s holds the last step for which ALL copy-engine
 * blocks of source s for expert group g have landed (written by a 4-byte peer copy that
 * follows the data copies in the same stream). A flag array therefore has
 * 2 * (BMOE_EP_MAX_GROUPS + 1) * ranks slots. */
#define BMOE_EP_COPY_FLAGS(ranks) ((BMOE_EP_MAX_GROUPS + 1u) * (ranks))

/* Routed rows per expert of this rank in one pass over its assignments:
 * counts_dev[id] (int64 [bins], zeroed here) += 1 for every assignment with a valid
 * expert id in [0, experts). With parts_dev / shard_base_dev (int64 [experts], row
 * shards of split experts) the id is shard_base[e] + i % parts[e] for assignment i and
 * bins is the number of shards; otherwise id = e and bins = experts. ids_out_dev
 * (int64 [assignments], may be NULL) receives the ids, -1 for dropped assignments.
 * bins <= 4096. */
int bmoe_ep_count(const int64_t* expert_ids_dev, uint64_t assignments, uint32_t experts,
                  const int64_t* parts_dev, const int64_t* shard_base_dev, uint32_t bins,
                  int64_t* ids_out_dev, int64_t* counts_dev, void* stream);

typedef struct bmoe_ep_plan_args {
  const int64_t* counts_all_dev;   /* [ranks, experts] routed rows per (source rank, expert),
                                      the all-gathered result of bmoe_ep_count */
  const int32_t* owner_dev;        /* [experts] owning rank */
  const int32_t* order_dev;        /* [experts] expert ids sorted by (owner, id) */
  int64_t* row_base_dev;           /* out [experts]: first row of (expert, this rank) in the
                                      owner's packed A */
  uint8_t* group_of_dev;           /* out [experts]: exchange group of the expert on its owner */
  uint8_t* group_local_dev;        /* out [experts of this rank], in packed order */
  uint32_t* expert_row_dev;        /* out [experts of this rank]: first packed row */
  uint32_t* local_rows_dev;        /* out [experts of this rank]: rows (the GEMM's counts) */
  uint32_t* bucket_offset_dev;     /* out [groups + 3], as bmoe_ep_route reads it */
  uint32_t* totals_dev;            /* out [2]: rows this rank owns in this step; 1 if that
                                      exceeds rows_cap (the step's results are then invalid) */
  uint64_t rows_cap;
  uint32_t experts;                /* <= 4096 */
  uint32_t ranks;
  uint32_t self;
  uint32_t groups;
  uint32_t tile_m;                 /* rows per tile of the grouped GEMM (group balance) */
  void* stream;
} bmoe_ep_plan_args;

/* Tables of one exchange step, derived on the device from the count matrix (one small
 * launch): where every (expert, source) block starts in its owner's packed A, the
 * exchange groups (contiguous runs of an owner's experts with about equal tile counts),
 * this rank's bucket sizes, and the rows per local expert. Same integer arithmetic as
 * the host planner of the Python layer; with it a step needs no host synchronisation.
 * No counterpart in the reference (it has no multi-GPU path). */
int bmoe_ep_plan(const bmoe_ep_plan_args* args);

typedef struct bmoe_ep_route_args {
  const int64_t* expert_ids_dev;   /* [assignments] expert of assignment i (token i / top_k);
                                      ids outside [0, experts) are dropped */
  const int64_t* row_base_dev;     /* [experts] first row of (expert, this rank) in the owner's A */
  const int32_t* owner_dev;        /* [experts] owning rank */
  const uint8_t* group_of_dev;     /* [experts] exchange group of the expert, < groups */
  uint32_t* cursor_dev;            /* [experts] zero at step start */
  void* const* origin_bases_dev;   /* [ranks] int64 origin record per packed row */
  void* entries_dev;               /* [assignments] 16-byte route entries, written here */
  const uint32_t* bucket_offset_dev; /* [groups + 3] first entry of bucket b: groups 0..G-1 hold
                                      the rows bound for other ranks, bucket G the rows that
                                      stay, bucket G + 1 the rows of copy-engine blocks (below);
                                      sizes follow from the count matrix */
  uint32_t* bucket_fill_dev;       /* [groups + 2] zero at step start */
  int32_t* dst_rank_out_dev;       /* [assignments] or NULL: destination of every assignment */
  int64_t* dst_row_out_dev;        /* [assignments] or NULL */
  uint64_t assignments;            /* < 2^32 */
  uint64_t rows_cap;               /* rows every packed A holds, < 2^32 */
  uint32_t top_k;
  uint32_t experts;
  uint32_t ranks;
  uint32_t self;
  uint32_t groups;
  void* stream;
  /* Copy-engine blocks (appended; NULL = none). staging_row_base_dev[e] >= 0 marks expert
   * e as one whose rows of this rank travel to the owner as ONE peer copy instead of
   * SM stores: its entries go to bucket G + 1 with this rank as destination and row
   * staging_row_base_dev[e] + position, i.e. into a local staging buffer in the order
   * the rows take in the owner's A (bmoe_ep_dispatch mode BMOE_EP_PACK fills it,
   * bmoe_peer_copy_batch sends it). The origin record is written as for any row. */
  const int64_t* staging_row_base_dev;  /* [experts] or NULL */
  uint64_t staging_rows_cap;
  /* Send-once mode (appended; NULL = every assignment sends its row). A token routed to
   * several experts of ONE other rank then crosses NVLink once: of its assignments to
   * that rank the one with the smallest (exchange group, position in the top-k list) is
   * the primary and is routed as before; the others get their row and origin record but
   * no route entry, and primary_out_dev[i] names the primary's assignment (-1: not a
   * duplicate). bmoe_ep_duplicates then tells the owner which rows to copy. Needs
   * dst_row_out_dev; excludes staging_row_base_dev. */
  int32_t* primary_out_dev;             /* [assignments] or NULL */
} bmoe_ep_route_args;

/* Route planning of one step: the destination row of every assignment (the row inside
 * (expert, source) comes from an atomic cursor, so the order of rows inside an expert
 * is arbitrary; no result row depends on it), the origin record
 * rank << 40 | assignment beside that row in the owner's memory, and one entry per
 * routed row in the bucket of its exchange group. Precedes bmoe_ep_dispatch in stream
 * order. */
int bmoe_ep_route(const bmoe_ep_route_args* args);

typedef struct bmoe_ep_duplicates_args {
  const int64_t* expert_ids_dev;   /* [assignments], as given to bmoe_ep_route */
  const int32_t* owner_dev;        /* [experts] */
  const uint8_t* group_of_dev;     /* [experts] */
  const int32_t* primary_dev;      /* [assignments] written by bmoe_ep_route */
  const int64_t* row_of_dev;       /* [assignments] bmoe_ep_route's dst_row_out_dev */
  void* const* record_bases_dev;   /* [ranks] record lists of every rank:
                                      uint32 pairs [groups][ranks][record_cap] */
  void* const* count_bases_dev;    /* [ranks] list lengths of every rank: uint32 [groups][ranks] */
  uint32_t* fill_dev;              /* [ranks * groups] zero at step start */
  uint32_t* done_counter_dev;      /* zero at step start */
  uint64_t assignments;
  uint32_t record_cap;             /* records one (group, source) list holds */
  uint32_t experts;
  uint32_t ranks;
  uint32_t self;
  uint32_t groups;
  void* stream;
} bmoe_ep_duplicates_args;

/* Send-once mode, after bmoe_ep_route and before the bmoe_ep_dispatch launch that raises
 * the flags, same stream: appends one record {packed row of the primary, packed row of the
 * duplicate} per duplicate assignment to list (group of the duplicate, this rank) in the
 * OWNER's memory and publishes the list lengths there. The owner's grouped GEMM copies
 * the rows itself (bmoe_plan_set_expand). No counterpart in the reference. */
int bmoe_ep_duplicates(const bmoe_ep_duplicates_args* args);

typedef struct bmoe_ep_dispatch_args {
  const void* x_dev;               /* [tokens, row_bytes] token rows of this rank */
  const void* entries_dev;         /* route entries written by bmoe_ep_route */
  const uint32_t* bucket_offset_dev; /* [groups + 2], as for bmoe_ep_route */
  void* const* a_bases_dev;        /* [ranks] packed A buffers, rows_cap rows each */
  void* const* flag_bases_dev;     /* [ranks] flag arrays (REMOTE / ALL with ranks > 1) */
  uint32_t* group_done_dev;        /* [groups] zero at step start (REMOTE / ALL) */
  uint32_t* chunk_next_dev;        /* [groups + 2] zero at step start */
  uint64_t assignments;            /* entries in all buckets together (sizes the grid) */
  uint64_t tokens;                 /* rows of x */
  uint64_t rows_cap;
  uint32_t row_bytes;              /* k * 2, multiple of 16 */
  uint32_t ranks;
  uint32_t self;
  uint32_t groups;
  uint32_t mode;                   /* BMOE_EP_LOCAL / REMOTE / ALL / PACK (PACK: bucket
                                      G + 1 only, a_bases_dev[self] = the staging buffer,
                                      rows_cap = its rows; raises no flag) */
  uint32_t epoch;
  uint32_t max_ctas;               /* 0 = default: 4 per SM for LOCAL, 7/16 of the SMs otherwise */
  uint32_t block_threads;          /* 0 = 256; 256, 512 or 1024 */
  uint32_t cluster;                /* 2 = launch the CTAs as pairs that fill whole SM pairs */
  uint32_t bulk_copies;            /* 1 = rows travel as TMA bulk copies through shared-memory
                                      stages (one row per warp, as many warps as fit in 220 KB,
                                      at most 16): for CTAs on SMs of their own */
  uint32_t* status_dev;            /* optional: 0x40000000 | bucket if a bulk-copy wait ran out */
  void* stream;
  const uint32_t* bucket_fill_dev; /* appended, optional [groups + 2]: entries bmoe_ep_route
                                      really wrote per bucket (its bucket_fill_dev); needed in
                                      send-once mode, where buckets are not filled to the end */
} bmoe_ep_dispatch_args;

/* Copies the routed token rows into the owners' packed A, bucket by bucket: REMOTE
 * walks the exchange groups in order and raises a group's flags on all peers when the
 * last CTA has finished it; LOCAL copies the rows that stay on this rank; ALL does
 * both (groups first). LOCAL and REMOTE launches of a step may overlap. */
int bmoe_ep_dispatch(const bmoe_ep_dispatch_args* args);

typedef struct bmoe_ep_return_args {
  const void* d_dev;               /* [rows, row_bytes] packed results of this rank */
  const void* origin_dev;          /* [rows] int64 origin records (this rank's own buffer) */
  void* const* y_bases_dev;        /* [ranks] result buffers in assignment order */
  void* const* flag_bases_dev;
  uint32_t* done_counter_dev;      /* zero at step start */
  uint64_t rows;
  uint64_t y_rows_cap;
  uint32_t row_bytes;              /* n * 2, multiple of 16 */
  uint32_t ranks;
  uint32_t self;
  uint32_t flag_slot;              /* BMOE_EP_MAX_GROUPS * ranks + self */
  uint32_t epoch;
  uint32_t max_ctas;               /* 0 = default */
  void* stream;
} bmoe_ep_return_args;

/* Writes every packed result row to row `assignment` of its origin rank's y and
 * then raises this rank's "done" flag on every peer. */
int bmoe_ep_return(const bmoe_ep_return_args* args);

/* Stream-ordered wait until slots first_slot + r (r != self) of the local flag
 * array have reached `epoch`. Bounded: after budget_ns (0 = 1 s) the kernel stores
 * 0x80000000 | first_slot << 8 | r in *status_dev (if it was 0) and returns. */
int bmoe_ep_wait_flags(const uint32_t* flags_dev, uint32_t first_slot, uint32_t ranks,
                       uint32_t self, uint32_t epoch, uint64_t budget_ns,
                       uint32_t* status_dev, void* stream);

/* Gate for the next bmoe_plan_run calls: the tile scheduler publishes a tile of
 * expert e only after slots group_of_expert[e]*ranks + r (all r != self) of the
 * local flag array reached `epoch` (bounded by the plan's wait budget; running out
 * reports BMOE_DEVICE_TIMEOUT through bmoe_plan_poll). flags_dev == NULL removes
 * the gate, and so does every bmoe_plan_initialize.
 * group_of_expert_dev: [experts of the plan] uint8, values < 32.
 * Forward progress: the flags must be raised by OTHER GPUs (or by copies, see below),
 * never by a kernel of this GPU that is launched separately: a persistent gated launch
 * may occupy every SM it is given, and nothing guarantees that another launch of the same
 * GPU runs beside it. Work of this GPU that the launch depends on (the rows that stay on
 * the rank) precedes it in stream order instead. A rank that pushes rows to its peers
 * from a kernel of its own while its gated GEMM runs should leave that kernel SMs the
 * GEMM's grid does not cover (cta_count below the SM count), otherwise every rank can end
 * up with a resident GEMM waiting for pushes that no peer has room to run; the wait is
 * bounded either way and reports BMOE_DEVICE_TIMEOUT. */
int bmoe_plan_set_gate(bmoe_plan* plan, const uint32_t* flags_dev, uint32_t epoch,
                       uint32_t ranks, uint32_t self, const uint8_t* group_of_expert_dev);

/* Extends the gate to rows that arrive as peer copies (copy-engine blocks): a tile of
 * group g is also held back until, for every source s whose bit is set in
 * copy_mask_dev[g], slot BMOE_EP_COPY_FLAGS(ranks) + g*ranks + s of the flag array given
 * to bmoe_plan_set_gate has reached the gate's epoch. copy_mask_dev: uint32 [groups of
 * this rank], NULL switches the extension off. Call after bmoe_plan_set_gate. No
 * counterpart in the reference (it has no multi-GPU path). */
int bmoe_plan_set_gate_copies(bmoe_plan* plan, const uint32_t* copy_mask_dev);

/* Send-once mode on the owner's side: the grouped GEMM itself copies duplicate rows.
 * One spare warp of every CTA walks, group by group, the record lists that the sources
 * wrote (bmoe_ep_duplicates) as soon as a source's flag for the group is up, copies
 * A[from] -> A[to] (both rows of this rank's packed A) and counts the copies in
 * done_dev[group]; the gate publishes a tile of a group only when all of the group's
 * records have been carried out. One launch, so no kernel of this GPU waits for another.
 *   records_dev  uint32 pairs [groups][ranks][record_cap]   (written by the peers)
 *   counts_dev   uint32 [groups][ranks]                     (written by the peers)
 *   next_dev     uint32 [groups][ranks]  claim counters, zero at step start
 *   done_dev     uint32 [groups]         zero at step start
 * Call after bmoe_plan_set_gate (same flags, epoch, ranks); records_dev == NULL switches
 * it off. a_dev / rows_cap / row_bytes describe the packed A buffer. */
int bmoe_plan_set_expand(bmoe_plan* plan, const void* records_dev, const uint32_t* counts_dev,
                         uint32_t* next_dev, uint32_t* done_dev, void* a_dev,
                         uint64_t rows_cap, uint32_t row_bytes, uint32_t record_cap,
                         uint32_t groups);

/* One device-to-device copy of a batch (bmoe_peer_copy_batch). */
typedef struct bmoe_copy_item {
  void* dst;        /* device pointer on any GPU mapped into this process */
  const void* src;
  uint64_t bytes;
  uint32_t stream;  /* index into the stream table */
  uint32_t reserved;
} bmoe_copy_item;

/* Enqueues `count` asynchronous copies, item i on streams[items[i].stream], in array
 * order, one cudaMemcpyAsync each (the copy engines move the bytes; no SM is used).
 * Used for the large (expert, source) blocks of the expert-parallel exchange and for the
 * 4-byte flag words that follow them. items and streams are host arrays. */
int bmoe_peer_copy_batch(const bmoe_copy_item* items, uint32_t count, void* const* streams,
                         uint32_t stream_count);

/* Result push for the next bmoe_plan_run calls (BF16 output only): the epilogue
 * writes every valid result row to row `assignment` of y_bases_dev[rank], following
 * the origin record rank << 40 | assignment of the row (origin_dev, indexed by packed
 * row: expert_row_dev[e] + row inside expert e), instead of storing it to D. With
 * peer buffers in y_bases_dev this is the expert-parallel combine exchange, spread
 * over the run time of the GEMM. Records whose rank or assignment is out of range
 * are skipped. origin_dev == NULL switches back to D; so does bmoe_plan_initialize.
 * After the run, bmoe_ep_return with rows == 0 raises the "done" flags. */
int bmoe_plan_set_push(bmoe_plan* plan, const void* origin_dev,
                       const uint32_t* expert_row_dev, void* const* y_bases_dev,
                       uint32_t ranks, uint64_t y_rows_cap);

/* Device buffers that other processes on the node can map (CUDA IPC):
 * bmoe_peer_alloc allocates `bytes` and writes a 64-byte handle; another process
 * passes that handle to bmoe_peer_open and gets a pointer valid on ITS device
 * (peer access over NVLink). bmoe_peer_close unmaps, bmoe_peer_free releases the
 * owner's allocation. */
int bmoe_peer_alloc(uint64_t bytes, void** ptr_out, uint8_t* handle_out);
int bmoe_peer_open(const uint8_t* handle, void** ptr_out);
int bmoe_peer_close(void* ptr);
int bmoe_peer_free(void* ptr);

/* Loads every kernel of the library on the current device now (CUDA loads a kernel's
 * module lazily at its first launch otherwise, which can take tens of milliseconds).
 * Call it before latency-critical work and before the first multi-GPU step, whose
 * bounded waits assume that all ranks launch within the wait budget. */
int bmoe_preload_kernels(void);

/* Library build information ("sm_100a", CUDA runtime version, ...). */
const char* bmoe_build_info(void);

#ifdef __cplusplus
} /* extern "C" */
#endif

#endif /* BMOE_B200_H_ */
