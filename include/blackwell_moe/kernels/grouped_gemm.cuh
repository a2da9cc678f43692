// BF16 grouped GEMM for routed MoE experts: for every expert e with M_e > 0,
//   D_e[M_e, n] = A_e[M_e, k] * B_e[n, k]^T     (FP32 accumulate, BF16 out).
//
// Source-compatible with the reference boundary
// include/blackwell_moe/kernels/grouped_gemm.cuh:10-71 (argument struct,
// status enum, plan class, one-shot launcher). Members added here are appended
// after the reference's and default to the reference behaviour. The plan is
// backed by the sm_100a engine behind the C interface in include/bmoe_b200.h.
#pragma once

#include <cstddef>
#include <cstdint>

#include "blackwell_moe/scheduler/scheduler.cuh"

namespace blackwell_moe {

enum class DataType { kBf16, kFp8E4M3 };

struct GroupedGemmArguments {
  // a, b, d: HOST arrays with `experts` entries, each a DEVICE pointer.
  //   a[e]: row-major [M_e, k]    b[e]: row-major [n, k]    d[e]: row-major [M_e, n]
  // Entries of experts without tokens may be null. All non-null pointers must
  // be 16-byte aligned. tokens_per_expert is a host array of `experts` counts.
  const void* const* a = nullptr;
  const void* const* b = nullptr;
  void* const* d = nullptr;
  const std::uint32_t* tokens_per_expert = nullptr;
  std::uint32_t experts = 0;
  std::uint32_t n = 0;
  std::uint32_t k = 0;
  DataType data_type = DataType::kBf16;
  SchedulerKind scheduler = SchedulerKind::kExpertOrder;
  // Default CUDA stream (a cudaStream_t passed opaquely).
  void* stream = nullptr;

  // ---- engine extensions; zero means "engine default" ----
  // Tiles claimed per atomic for kDynamicQueue (default 1).
  std::uint32_t claim_size = 0;
  // kDynamicQueue only: the last `hybrid_tail_tiles` tiles are claimed one at a
  // time from a second counter, the rest in chunks of claim_size.
  std::uint32_t hybrid_tail_tiles = 0;
  // Persistent scheduling units to launch: CTAs, or CTA pairs when cta_group
  // is 2 (default: one CTA per SM). Ignored by kClc.
  std::uint32_t cta_count = 0;
  // Output tile width: 128 or 256 (default 256). Tile height is 128 per CTA.
  std::uint32_t tile_n = 0;
  // 1 = one CTA computes a 128-row tile; 2 = two CTAs of a cluster compute a
  // 256 x 256 tile together; 0 = the engine picks (pairs unless 256-row tiles
  // would pad the routed rows by more than 10 % over 128-row tiles).
  std::uint32_t cta_group = 0;
  // 0 = worklist in the reference order (tile_n fastest); 1 = tile_m fastest
  // inside each expert, which keeps the expert's rows in L2 while its weights
  // stream once (default 1).
  std::int32_t raster_along_m = -1;
};

enum class KernelStatus {
  kSuccess,
  kInvalidArgument,
  kUnsupportedDataType,
  kUnsupportedScheduler,
  kUnsupportedDevice,
  kCudaError,
  kCutlassError,   // kept for ordinal compatibility; never returned
  kDeviceTimeout,  // a bounded in-kernel wait expired; see Bf16GroupedGemmPlan::poll()
};

const char* kernel_status_string(KernelStatus status);

struct GroupedGemmPlanStats {
  std::uint32_t active_experts = 0;
  std::uint32_t threadblock_count = 0;
  std::size_t workspace_bytes = 0;
  // ---- engine extensions ----
  std::uint32_t total_tiles = 0;
  std::uint32_t tile_m = 0;
  std::uint32_t tile_n = 0;
  SchedulerKind resolved_scheduler = SchedulerKind::kExpertOrder;
  std::uint32_t claim_size = 0;
  std::uint32_t hybrid_tail_tiles = 0;
};

// Reusable launch plan. initialize() validates, builds the device worklist and
// the per-expert TMA descriptors (it may allocate and copy); run() only
// launches. Re-initialising an existing plan releases or reuses its storage.
class Bf16GroupedGemmPlan {
 public:
  Bf16GroupedGemmPlan();
  ~Bf16GroupedGemmPlan();

  Bf16GroupedGemmPlan(const Bf16GroupedGemmPlan&) = delete;
  Bf16GroupedGemmPlan& operator=(const Bf16GroupedGemmPlan&) = delete;
  Bf16GroupedGemmPlan(Bf16GroupedGemmPlan&& other) noexcept;
  Bf16GroupedGemmPlan& operator=(Bf16GroupedGemmPlan&& other) noexcept;

  KernelStatus initialize(const GroupedGemmArguments& args);
  // Asynchronous: returns after enqueueing on `stream` (or the plan default).
  KernelStatus run(void* stream = nullptr);
  GroupedGemmPlanStats stats() const;

  // Extension: synchronises the plan's last stream and reports
  // kDeviceTimeout if any launch since initialize() gave up on a bounded wait.
  KernelStatus poll();
  // Extension: the underlying C handle (bmoe_plan*), for mixed C/C++ callers.
  void* native_handle() const;
  // Extensions for the expert-parallel exchange (no counterpart in the reference).
  // Both apply to the next run() calls and are cleared by initialize().
  // Gate: a tile of expert e is scheduled only after the flag slots
  // group_of_expert[e] * ranks + r (r != self) have reached `epoch`; a null
  // `flags` removes the gate. All pointers are device pointers.
  KernelStatus set_exchange_gate(const std::uint32_t* flags, std::uint32_t epoch,
                                 std::uint32_t ranks, std::uint32_t self,
                                 const std::uint8_t* group_of_expert);
  // Push: result rows go to row `assignment` of y_bases[rank] following the
  // origin record (rank << 40 | assignment) of each packed row instead of D;
  // a null `origin` switches back to D.
  KernelStatus set_result_push(const void* origin, const std::uint32_t* expert_first_row,
                               void* const* y_bases, std::uint32_t ranks,
                               std::uint64_t y_rows_cap);

 private:
  friend class Fp8E4m3GroupedGemmPlan;
  KernelStatus initialize_typed(const GroupedGemmArguments& args);
  struct Impl;
  Impl* impl_ = nullptr;
};

// Extension: the same plan over FP8 E4M3 operands (one byte per element, no scales):
//   D_e[M_e, n] = float(A_e)[M_e, k] * float(B_e)[n, k]^T    (FP32 accumulate, BF16 out)
// The reference declares DataType::kFp8E4M3 (grouped_gemm.cuh:10) and rejects it
// everywhere (baselines/cutlass/cutlass_baseline.cu:211-213); Bf16GroupedGemmPlan keeps
// that behaviour, this class is where the type is accepted. args.data_type must be
// kFp8E4M3 (anything else: kUnsupportedDataType) and k a multiple of 16.
class Fp8E4m3GroupedGemmPlan {
 public:
  KernelStatus initialize(const GroupedGemmArguments& args);
  KernelStatus run(void* stream = nullptr) { return plan_.run(stream); }
  GroupedGemmPlanStats stats() const { return plan_.stats(); }
  KernelStatus poll() { return plan_.poll(); }
  void* native_handle() const { return plan_.native_handle(); }

 private:
  Bf16GroupedGemmPlan plan_;
};

// One-shot convenience path (plan, initialize, run). Benchmarks reuse a plan.
KernelStatus launch_grouped_gemm_baseline(const GroupedGemmArguments& args);

}  // namespace blackwell_moe
