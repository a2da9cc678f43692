"""ctypes binding of the engine's C interface (``include/bmoe_b200.h``).

The shared library is the product: loading fails loudly when it has not been
built, and nothing here falls back to a CPU implementation.
"""

from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
# BMOE_CHECKS=1 in the environment selects the bounds-checked build of the same sources
# (python -m ... _build --checks, or __graft_entry__.build()).
LIB_PATH = PKG_DIR / "lib" / ("libbmoe_b200_checks.so" if os.environ.get("BMOE_CHECKS") == "1"
                              else "libbmoe_b200.so")

# ---- status codes / enums (bmoe_b200.h) ----
OK = 0
INVALID_ARGUMENT = 1
UNSUPPORTED_DATA_TYPE = 2
UNSUPPORTED_SCHEDULER = 3
UNSUPPORTED_DEVICE = 4
CUDA_ERROR = 5
BACKEND_ERROR = 6
DEVICE_TIMEOUT = 7

SCHED_EXPERT_ORDER = 0
SCHED_STATIC_PERSISTENT = 1
SCHED_DYNAMIC_QUEUE = 2
SCHED_COMPACTED = 3
SCHED_AUTO = 4
SCHED_CLC = 5

SCHEDULER_NAMES = {
    "expert_order": SCHED_EXPERT_ORDER,
    "baseline": SCHED_EXPERT_ORDER,
    "static": SCHED_STATIC_PERSISTENT,
    "static_persistent": SCHED_STATIC_PERSISTENT,
    "sorted_static": SCHED_STATIC_PERSISTENT,
    "dynamic": SCHED_DYNAMIC_QUEUE,
    "dynamic_queue": SCHED_DYNAMIC_QUEUE,
    "compacted": SCHED_COMPACTED,
    "auto": SCHED_AUTO,
    "clc": SCHED_CLC,
    "clc_assisted": SCHED_CLC,
}

WORKLIST_STATIC_MAX_EXPERTS = 1024

ORDER_EXPERT = 0
ORDER_SORTED_BY_WORK = 1
RASTER_N_FASTEST = 0
RASTER_M_FASTEST = 1

DISTRIBUTIONS = {"uniform": 0, "heavy_hitter": 1, "heavy": 1, "sparse": 2, "zipf": 3,
                 "heavy_sparse": 4}

VARIANT_NAMES = (
    "v0_nonpersistent",
    "v1_static_ws",
    "v2_dynamic",
    "v3_chunked",
    "v4_hybrid",
    "v5_clc",
)


class Tile(C.Structure):
    _fields_ = [
        ("expert_id", C.c_uint32),
        ("tile_m", C.c_uint32),
        ("tile_n", C.c_uint32),
        ("valid_m", C.c_uint32),
        ("valid_n", C.c_uint32),
    ]


class WorkloadConfig(C.Structure):
    _fields_ = [
        ("experts", C.c_uint32),
        ("distribution", C.c_uint32),
        ("total_tokens", C.c_uint64),
        ("seed", C.c_uint64),
        ("zipf_alpha", C.c_double),
        ("heavy_hitter_fraction", C.c_double),
        ("heavy_hitter_token_share", C.c_double),
        ("inactive_expert_fraction", C.c_double),
    ]


class WorkloadMetrics(C.Structure):
    _fields_ = [
        ("mean_tokens", C.c_double),
        ("coefficient_of_variation", C.c_double),
        ("max_over_mean", C.c_double),
        ("inactive_expert_ratio", C.c_double),
        ("small_m_expert_ratio", C.c_double),
        ("tile_count_cv", C.c_double),
        ("active_experts", C.c_uint32),
        ("reserved", C.c_uint32),
        ("total_tiles", C.c_uint64),
    ]


class ScheduleMetrics(C.Structure):
    _fields_ = [
        ("total_tiles", C.c_uint64),
        ("total_valid_elements", C.c_uint64),
        ("total_padded_elements", C.c_uint64),
        ("expert_switches", C.c_uint64),
        ("min_tiles_per_cta", C.c_uint64),
        ("max_tiles_per_cta", C.c_uint64),
        ("mean_cta_work", C.c_double),
        ("max_cta_work", C.c_double),
        ("cta_work_cv", C.c_double),
        ("tail_ratio", C.c_double),
        ("estimated_utilization", C.c_double),
        ("useful_work_ratio", C.c_double),
    ]


class RoutingFeatures(C.Structure):
    _fields_ = [
        ("mean_m", C.c_double),
        ("cv_m", C.c_double),
        ("max_over_mean_m", C.c_double),
        ("inactive_expert_ratio", C.c_double),
        ("small_m_expert_ratio", C.c_double),
        ("expert_tile_cv", C.c_double),
        ("max_expert_tiles_over_mean", C.c_double),
        ("active_tiles", C.c_uint64),
        ("tiles_per_cta", C.c_double),
        ("useful_work_ratio", C.c_double),
    ]


class EpRouteArgs(C.Structure):
    _fields_ = [
        ("expert_ids_dev", C.c_void_p), ("row_base_dev", C.c_void_p), ("owner_dev", C.c_void_p),
        ("group_of_dev", C.c_void_p), ("cursor_dev", C.c_void_p),
        ("origin_bases_dev", C.c_void_p), ("entries_dev", C.c_void_p),
        ("bucket_offset_dev", C.c_void_p), ("bucket_fill_dev", C.c_void_p),
        ("dst_rank_out_dev", C.c_void_p), ("dst_row_out_dev", C.c_void_p),
        ("assignments", C.c_uint64), ("rows_cap", C.c_uint64),
        ("top_k", C.c_uint32), ("experts", C.c_uint32), ("ranks", C.c_uint32),
        ("self", C.c_uint32), ("groups", C.c_uint32),
        ("stream", C.c_void_p),
        ("staging_row_base_dev", C.c_void_p), ("staging_rows_cap", C.c_uint64),
        ("primary_out_dev", C.c_void_p),
    ]


class EpDuplicatesArgs(C.Structure):
    _fields_ = [
        ("expert_ids_dev", C.c_void_p), ("owner_dev", C.c_void_p), ("group_of_dev", C.c_void_p),
        ("primary_dev", C.c_void_p), ("row_of_dev", C.c_void_p),
        ("record_bases_dev", C.c_void_p), ("count_bases_dev", C.c_void_p),
        ("fill_dev", C.c_void_p), ("done_counter_dev", C.c_void_p),
        ("assignments", C.c_uint64), ("record_cap", C.c_uint32), ("experts", C.c_uint32),
        ("ranks", C.c_uint32), ("self", C.c_uint32), ("groups", C.c_uint32),
        ("stream", C.c_void_p),
    ]


class EpPlanArgs(C.Structure):
    _fields_ = [
        ("counts_all_dev", C.c_void_p), ("owner_dev", C.c_void_p), ("order_dev", C.c_void_p),
        ("row_base_dev", C.c_void_p), ("group_of_dev", C.c_void_p),
        ("group_local_dev", C.c_void_p), ("expert_row_dev", C.c_void_p),
        ("local_rows_dev", C.c_void_p), ("bucket_offset_dev", C.c_void_p),
        ("totals_dev", C.c_void_p), ("rows_cap", C.c_uint64),
        ("experts", C.c_uint32), ("ranks", C.c_uint32), ("self", C.c_uint32),
        ("groups", C.c_uint32), ("tile_m", C.c_uint32),
        ("stream", C.c_void_p),
    ]


class CopyItem(C.Structure):
    _fields_ = [("dst", C.c_void_p), ("src", C.c_void_p), ("bytes", C.c_uint64),
                ("stream", C.c_uint32), ("reserved", C.c_uint32)]


COPY_ITEM_DTYPE = [("dst", "<u8"), ("src", "<u8"), ("bytes", "<u8"), ("stream", "<u4"),
                   ("reserved", "<u4")]


class EpDispatchArgs(C.Structure):
    _fields_ = [
        ("x_dev", C.c_void_p), ("entries_dev", C.c_void_p), ("bucket_offset_dev", C.c_void_p),
        ("a_bases_dev", C.c_void_p), ("flag_bases_dev", C.c_void_p),
        ("group_done_dev", C.c_void_p), ("chunk_next_dev", C.c_void_p),
        ("assignments", C.c_uint64), ("tokens", C.c_uint64), ("rows_cap", C.c_uint64),
        ("row_bytes", C.c_uint32), ("ranks", C.c_uint32), ("self", C.c_uint32),
        ("groups", C.c_uint32), ("mode", C.c_uint32), ("epoch", C.c_uint32),
        ("max_ctas", C.c_uint32), ("block_threads", C.c_uint32), ("cluster", C.c_uint32),
        ("bulk_copies", C.c_uint32), ("status_dev", C.c_void_p),
        ("stream", C.c_void_p),
        ("bucket_fill_dev", C.c_void_p),
    ]


class EpReturnArgs(C.Structure):
    _fields_ = [
        ("d_dev", C.c_void_p), ("origin_dev", C.c_void_p), ("y_bases_dev", C.c_void_p),
        ("flag_bases_dev", C.c_void_p), ("done_counter_dev", C.c_void_p),
        ("rows", C.c_uint64), ("y_rows_cap", C.c_uint64),
        ("row_bytes", C.c_uint32), ("ranks", C.c_uint32), ("self", C.c_uint32),
        ("flag_slot", C.c_uint32), ("epoch", C.c_uint32), ("max_ctas", C.c_uint32),
        ("stream", C.c_void_p),
    ]


EP_MAX_GROUPS = 16
EP_LOCAL, EP_REMOTE, EP_ALL, EP_PACK = 0, 1, 2, 3


def ep_copy_flags(ranks: int) -> int:
    """First slot of the flag plane for rows that arrive as peer copies."""
    return (EP_MAX_GROUPS + 1) * ranks


class WorklistTotals(C.Structure):
    _fields_ = [
        ("total_tiles", C.c_uint32),
        ("active_experts", C.c_uint32),
        ("total_rows", C.c_uint64),
        ("total_valid_elements", C.c_uint64),
        ("overflow", C.c_uint32),
        ("reserved", C.c_uint32),
    ]


class WorklistLayout(C.Structure):
    _fields_ = [
        ("bytes", C.c_size_t),
        ("off_totals", C.c_size_t),
        ("off_row_offsets", C.c_size_t),
        ("off_expert_m_tiles", C.c_size_t),
        ("off_expert_tiles", C.c_size_t),
        ("off_tile_offsets", C.c_size_t),
        ("off_active_ids", C.c_size_t),
        ("off_visit_order", C.c_size_t),
        ("off_visit_tile_offsets", C.c_size_t),
    ]


class WorklistRequest(C.Structure):
    _fields_ = [
        ("experts", C.c_uint32),
        ("n", C.c_uint32),
        ("tile_m", C.c_uint32),
        ("tile_n", C.c_uint32),
        ("order", C.c_uint32),
        ("raster", C.c_uint32),
    ]


class GemmArgs(C.Structure):
    _fields_ = [
        ("a", C.POINTER(C.c_void_p)),
        ("b", C.POINTER(C.c_void_p)),
        ("d", C.POINTER(C.c_void_p)),
        ("tokens_per_expert", C.POINTER(C.c_uint32)),
        ("experts", C.c_uint32),
        ("n", C.c_uint32),
        ("k", C.c_uint32),
        ("data_type", C.c_uint32),
        ("scheduler", C.c_uint32),
        ("claim_size", C.c_uint32),
        ("hybrid_tail_tiles", C.c_uint32),
        ("cta_count", C.c_uint32),
        ("tile_n", C.c_uint32),
        ("cta_group", C.c_uint32),
        ("raster_along_m", C.c_int32),
        ("output_f32", C.c_uint32),
        ("stream", C.c_void_p),
        ("packed_a", C.c_void_p),
        ("packed_rows", C.c_uint64),
        ("results_pushed", C.c_uint32),
        ("reserved0", C.c_uint32),
        ("tokens_per_expert_dev", C.c_void_p),
    ]


class PlanStats(C.Structure):
    _fields_ = [
        ("active_experts", C.c_uint32),
        ("threadblock_count", C.c_uint32),
        ("workspace_bytes", C.c_uint64),
        ("total_tiles", C.c_uint32),
        ("tile_m", C.c_uint32),
        ("tile_n", C.c_uint32),
        ("resolved_scheduler", C.c_uint32),
        ("claim_size", C.c_uint32),
        ("hybrid_tail_tiles", C.c_uint32),
        ("cta_group", C.c_uint32),
        ("stages", C.c_uint32),
        ("dynamic_smem_bytes", C.c_uint32),
        ("launches", C.c_uint32),
        ("sm_count", C.c_uint32),
    ]


class DeviceReport(C.Structure):
    _fields_ = [
        ("code", C.c_uint32),
        ("cta", C.c_uint32),
        ("role", C.c_uint32),
        ("tile", C.c_uint32),
        ("stage", C.c_uint32),
        ("aux", C.c_uint32),
        ("count", C.c_uint32),
        ("reserved", C.c_uint32),
    ]


class ProbeArgs(C.Structure):
    _fields_ = [
        ("tiles", C.c_void_p),
        ("tile_count", C.c_uint32),
        ("cta_count", C.c_uint32),
        ("claim_size", C.c_uint32),
        ("work_scale", C.c_uint32),
        ("next_tile", C.c_void_p),
        ("tile_visits", C.c_void_p),
        ("tile_checksums", C.c_void_p),
        ("cta_tile_counts", C.c_void_p),
        ("cta_valid_elements", C.c_void_p),
        ("stream", C.c_void_p),
    ]


_P = C.POINTER
_u32p = _P(C.c_uint32)

# name -> (restype, argtypes); every function declared in bmoe_b200.h.
SIGNATURES = {
    "bmoe_status_string": (C.c_char_p, [C.c_int]),
    "bmoe_generate_workload": (C.c_int, [_P(WorkloadConfig), _u32p]),
    "bmoe_workload_metrics_compute": (
        C.c_int,
        [_u32p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, _P(WorkloadMetrics)],
    ),
    "bmoe_host_tile_count": (
        C.c_uint64,
        [_u32p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32],
    ),
    "bmoe_host_build_tiles": (
        C.c_int,
        [_u32p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32,
         _P(Tile), C.c_uint64, _P(C.c_uint64)],
    ),
    "bmoe_host_simulate": (
        C.c_int,
        [C.c_uint32, _u32p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32,
         _P(Tile), C.c_uint64, _P(C.c_uint64), _P(ScheduleMetrics)],
    ),
    "bmoe_routing_features_compute": (
        C.c_int,
        [_u32p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32,
         _P(RoutingFeatures)],
    ),
    "bmoe_select_variant": (C.c_int, [_P(RoutingFeatures), _P(C.c_double), _u32p]),
    "bmoe_select_variant_fitted": (C.c_int, [_P(RoutingFeatures), _P(C.c_double), _u32p]),
    "bmoe_variant_name": (C.c_char_p, [C.c_uint32]),
    "bmoe_worklist_layout_for": (C.c_int, [C.c_uint32, _P(WorklistLayout)]),
    "bmoe_worklist_build": (
        C.c_int,
        [C.c_void_p, _P(WorklistRequest), C.c_void_p, C.c_uint32, C.c_void_p, C.c_void_p],
    ),
    "bmoe_worklist_build_static": (
        C.c_int,
        [C.c_void_p, _P(WorklistRequest), C.c_void_p, C.c_uint32, C.c_void_p, C.c_void_p],
    ),
    "bmoe_plan_create": (C.c_void_p, []),
    "bmoe_plan_destroy": (None, [C.c_void_p]),
    "bmoe_plan_initialize": (C.c_int, [C.c_void_p, _P(GemmArgs)]),
    "bmoe_plan_run": (C.c_int, [C.c_void_p, C.c_void_p]),
    "bmoe_plan_stats_get": (C.c_int, [C.c_void_p, _P(PlanStats)]),
    "bmoe_plan_poll": (C.c_int, [C.c_void_p, _P(DeviceReport)]),
    "bmoe_plan_read_worklist": (C.c_int, [C.c_void_p, _P(Tile), C.c_uint32, _u32p]),
    "bmoe_plan_set_observers": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p]),
    "bmoe_plan_set_trace": (C.c_int, [C.c_void_p, C.c_void_p]),
    "bmoe_grouped_gemm": (C.c_int, [_P(GemmArgs)]),
    "bmoe_probe_launch": (C.c_int, [C.c_uint32, _P(ProbeArgs)]),
    "bmoe_probe_scheduler_name": (C.c_char_p, [C.c_uint32]),
    "bmoe_ep_place_experts": (
        C.c_int,
        [_u32p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32,
         _u32p, _P(C.c_uint64)],
    ),
    "bmoe_gather_rows": (
        C.c_int,
        [C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint64, C.c_uint64, C.c_uint32, C.c_void_p],
    ),
    "bmoe_route_rows": (
        C.c_int,
        [C.c_void_p, C.c_uint32, C.c_uint64, C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32,
         C.c_uint64, C.c_void_p, C.c_void_p, C.c_uint64, C.c_uint32, C.c_uint32, C.c_void_p],
    ),
    "bmoe_combine_topk": (
        C.c_int,
        [C.c_void_p, C.c_uint32, C.c_uint64, C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint64,
         C.c_uint32, C.c_uint32, C.c_void_p, C.c_uint32, C.c_void_p],
    ),
    "bmoe_ep_count": (
        C.c_int,
        [C.c_void_p, C.c_uint64, C.c_uint32, C.c_void_p, C.c_void_p, C.c_uint32, C.c_void_p,
         C.c_void_p, C.c_void_p],
    ),
    "bmoe_ep_plan": (C.c_int, [C.c_void_p]),
    "bmoe_ep_route": (C.c_int, [C.c_void_p]),
    "bmoe_ep_duplicates": (C.c_int, [C.c_void_p]),
    "bmoe_ep_dispatch": (C.c_int, [C.c_void_p]),
    "bmoe_ep_return": (C.c_int, [C.c_void_p]),
    "bmoe_ep_wait_flags": (
        C.c_int,
        [C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint64, C.c_void_p,
         C.c_void_p],
    ),
    "bmoe_plan_set_gate": (
        C.c_int, [C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_void_p]),
    "bmoe_plan_set_gate_copies": (C.c_int, [C.c_void_p, C.c_void_p]),
    "bmoe_plan_set_expand": (
        C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                  C.c_uint64, C.c_uint32, C.c_uint32, C.c_uint32]),
    "bmoe_peer_copy_batch": (C.c_int, [C.c_void_p, C.c_uint32, C.c_void_p, C.c_uint32]),
    "bmoe_plan_set_push": (
        C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint64]),
    "bmoe_peer_alloc": (C.c_int, [C.c_uint64, _P(C.c_void_p), C.c_void_p]),
    "bmoe_peer_open": (C.c_int, [C.c_void_p, _P(C.c_void_p)]),
    "bmoe_peer_close": (C.c_int, [C.c_void_p]),
    "bmoe_peer_free": (C.c_int, [C.c_void_p]),
    "bmoe_preload_kernels": (C.c_int, []),
    "bmoe_build_info": (C.c_char_p, []),
}

_lib = None


def load() -> C.CDLL:
    """Load ``libbmoe_b200.so`` and declare every entry point."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with "
            "`python __graft_entry__.py` (nvcc, sm_100a). There is no CPU fallback."
        )
    lib = C.CDLL(str(LIB_PATH))
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is not exported
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def status_string(status: int) -> str:
    return load().bmoe_status_string(int(status)).decode()


class EngineError(RuntimeError):
    """A C entry point returned a non-zero status."""

    def __init__(self, status: int, where: str):
        self.status = int(status)
        super().__init__(f"{where}: {status_string(status)} (status {status})")


def check(status: int, where: str) -> None:
    if status != OK:
        raise EngineError(status, where)
