"""Python face of the sm_100a engine: plan, device worklist builder, probe.

Everything here calls the C interface (``include/bmoe_b200.h``); PyTorch is
used only to own device memory and streams. Names follow the reference's C++
boundary (``Bf16GroupedGemmPlan``: ``initialize`` / ``run`` / ``stats``,
include/blackwell_moe/kernels/grouped_gemm.cuh:51-69) and return the same
status codes instead of raising.
"""

from __future__ import annotations

import ctypes as C
from typing import Sequence

import numpy as np

from . import _capi

TILE_DTYPE = np.dtype(
    [("expert_id", "<u4"), ("tile_m", "<u4"), ("tile_n", "<u4"),
     ("valid_m", "<u4"), ("valid_n", "<u4")]
)


def _scheduler_id(scheduler) -> int:
    if isinstance(scheduler, str):
        if scheduler not in _capi.SCHEDULER_NAMES:
            raise ValueError(f"unknown scheduler: {scheduler}")
        return _capi.SCHEDULER_NAMES[scheduler]
    return int(scheduler)


def _stream_ptr(stream) -> int | None:
    if stream is None:
        return None
    if hasattr(stream, "cuda_stream"):
        return int(stream.cuda_stream) or None
    return int(stream) or None


def tiles_to_numpy(tiles, count: int) -> np.ndarray:
    """ctypes ``Tile`` array -> structured numpy array (copy)."""
    raw = np.frombuffer(tiles, dtype=TILE_DTYPE, count=count)
    return raw.copy()


class GroupedGemmPlan:
    """Reusable launch plan for ``D_e = A_e @ B_e^T`` over routed experts."""

    def __init__(self) -> None:
        self._lib = _capi.load()
        self._handle = self._lib.bmoe_plan_create()
        if not self._handle:
            raise MemoryError("bmoe_plan_create failed")
        self._keep = None  # argument arrays / tensors kept alive for the plan

    def close(self) -> None:
        if getattr(self, "_handle", None):
            self._lib.bmoe_plan_destroy(self._handle)
            self._handle = None

    def __del__(self) -> None:  # pragma: no cover - interpreter shutdown order
        try:
            self.close()
        except Exception:
            pass

    # ------------------------------------------------------------ set-up --
    def initialize(
        self,
        a_ptrs: Sequence[int],
        b_ptrs: Sequence[int],
        d_ptrs: Sequence[int],
        tokens_per_expert: Sequence[int],
        n: int,
        k: int,
        *,
        scheduler="expert_order",
        data_type: int = 0,
        stream=None,
        claim_size: int = 0,
        hybrid_tail_tiles: int = 0,
        cta_count: int = 0,
        tile_n: int = 0,
        cta_group: int = 0,
        raster_along_m: int = -1,
        output_f32: bool = False,
        packed_a: int = 0,
        packed_rows: int = 0,
        results_pushed: bool = False,
        tokens_per_expert_dev: int = 0,
    ) -> int:
        """Pointer-array form of the reference arguments. Returns a status.
        ``packed_a`` / ``packed_rows``: base and row capacity of ONE buffer holding all
        experts' rows back to back (one tensor map instead of one per expert; ``a_ptrs``
        is then ignored). ``results_pushed``: no D descriptors, results leave through
        ``set_push``."""
        experts = len(tokens_per_expert)

        def pointers(values):
            if isinstance(values, np.ndarray):
                arr = np.ascontiguousarray(values, dtype=np.uint64)
            else:
                arr = np.array([int(p or 0) for p in values], dtype=np.uint64)
            return arr if arr.size else np.zeros(1, dtype=np.uint64)

        arr_a, arr_b, arr_d = pointers(a_ptrs), pointers(b_ptrs), pointers(d_ptrs)
        counts = np.ascontiguousarray(tokens_per_expert, dtype=np.uint32)
        if counts.size == 0:
            counts = np.zeros(1, dtype=np.uint32)
        args = _capi.GemmArgs(
            a=arr_a.ctypes.data_as(C.POINTER(C.c_void_p)),
            b=arr_b.ctypes.data_as(C.POINTER(C.c_void_p)),
            d=arr_d.ctypes.data_as(C.POINTER(C.c_void_p)),
            tokens_per_expert=counts.ctypes.data_as(C.POINTER(C.c_uint32)),
            experts=experts,
            n=n,
            k=k,
            data_type=data_type,
            scheduler=_scheduler_id(scheduler),
            claim_size=claim_size,
            hybrid_tail_tiles=hybrid_tail_tiles,
            cta_count=min(int(cta_count), 0xFFFFFFFF),
            tile_n=tile_n,
            cta_group=cta_group,
            raster_along_m=raster_along_m,
            output_f32=1 if output_f32 else 0,
            stream=_stream_ptr(stream),
            packed_a=int(packed_a) or None,
            packed_rows=int(packed_rows),
            results_pushed=1 if results_pushed else 0,
            reserved0=0,
            tokens_per_expert_dev=int(tokens_per_expert_dev) or None,
        )
        return int(self._lib.bmoe_plan_initialize(self._handle, C.byref(args)))

    def initialize_packed(self, a, w, d, tokens_per_expert: Sequence[int], *,
                          single_a_map: bool = False, **options) -> int:
        """Packed form: ``a`` [sum M, k], ``w`` [E, n, k], ``d`` [sum M, n] CUDA
        tensors, rows of expert 0 first; ``a`` and ``w`` BF16, or both one byte per element
        (FP8 E4M3 bit patterns; k then a multiple of 16), ``d`` BF16 (FP32 with
        ``output_f32``). Row offsets are the exclusive prefix sum
        of the counts; every expert's slice starts on a 16-byte boundary because
        k and n are multiples of 8. ``single_a_map``: one tensor map over the whole of
        ``a`` instead of one per expert (cheaper to re-plan; tiles at an expert's ragged
        edge then also load the next expert's rows, which costs bandwidth when experts
        have few rows and changes no result)."""
        experts = len(tokens_per_expert)
        n, k = int(w.shape[1]), int(w.shape[2])
        d_elem = 4 if options.get("output_f32") else 2
        if d.element_size() != d_elem:
            return _capi.INVALID_ARGUMENT
        if int(w.shape[0]) != experts or int(a.shape[1]) != k or int(d.shape[1]) != n:
            return _capi.INVALID_ARGUMENT
        if not (a.is_contiguous() and w.is_contiguous() and d.is_contiguous()):
            return _capi.INVALID_ARGUMENT
        counts = np.asarray(tokens_per_expert, dtype=np.int64)
        total = int(counts.sum())
        if int(a.shape[0]) < total or int(d.shape[0]) < total:
            return _capi.INVALID_ARGUMENT
        first_row = (np.cumsum(counts) - counts).astype(np.uint64)
        elem = int(a.element_size())
        if elem != int(w.element_size()) or elem not in (1, 2):
            return _capi.INVALID_ARGUMENT
        if elem == 1:
            options["data_type"] = 1          # FP8 E4M3 bytes (torch.float8_e4m3fn or uint8)
        a_ptrs = np.uint64(a.data_ptr()) + first_row * np.uint64(k * elem)
        b_ptrs = (np.uint64(w.data_ptr()) +
                  np.arange(experts, dtype=np.uint64) * np.uint64(n * k * elem))
        d_ptrs = np.uint64(d.data_ptr()) + first_row * np.uint64(n * d_elem)
        self._keep = (a, w, d)
        if single_a_map:
            options.update(packed_a=a.data_ptr(), packed_rows=int(a.shape[0]))
        return self.initialize(a_ptrs, b_ptrs, d_ptrs, counts, n, k, **options)

    def initialize_packed_device_counts(self, a, w, counts_dev_ptr: int, **options) -> int:
        """Packed form whose counts exist only on the device: ``counts_dev_ptr`` points at
        uint32 [E] rows per expert, written by work that precedes this call in the stream
        (for example ``bmoe_ep_plan``). Nothing is read back: the worklist is built from
        the device counts, the kernel takes the tile total from device memory, the grid is
        the full persistent grid, and the results leave through ``set_push``. ``a`` is
        the packed row buffer (its row count is the capacity)."""
        experts = int(w.shape[0])
        n, k = int(w.shape[1]), int(w.shape[2])
        if experts == 0 or int(a.shape[1]) != k or not (a.is_contiguous() and w.is_contiguous()):
            return _capi.INVALID_ARGUMENT
        b_ptrs = np.uint64(w.data_ptr()) + np.arange(experts, dtype=np.uint64) * np.uint64(n * k * 2)
        zeros = np.zeros(experts, dtype=np.uint64)
        self._keep = (a, w)
        return self.initialize(zeros, b_ptrs, zeros, np.zeros(experts, dtype=np.uint32), n, k,
                               packed_a=a.data_ptr(), packed_rows=int(a.shape[0]),
                               results_pushed=True, tokens_per_expert_dev=counts_dev_ptr,
                               **options)

    # --------------------------------------------------------------- run --
    def run(self, stream=None) -> int:
        return int(self._lib.bmoe_plan_run(self._handle, _stream_ptr(stream)))

    def set_gate(self, flags_ptr, epoch: int, ranks: int, self_rank: int, group_of_ptr) -> int:
        """Hold back the tiles of an expert group until the other ranks' rows of that
        group have arrived (see ``bmoe_plan_set_gate``); ``flags_ptr`` None removes it."""
        return int(self._lib.bmoe_plan_set_gate(self._handle, flags_ptr, epoch, ranks, self_rank,
                                                group_of_ptr))

    def set_gate_copies(self, copy_mask_ptr) -> int:
        """Also hold a group's tiles back until the sources in ``copy_mask[group]`` have
        raised the flags of their peer copies (``bmoe_plan_set_gate_copies``)."""
        return int(self._lib.bmoe_plan_set_gate_copies(self._handle, copy_mask_ptr or None))

    def set_expand(self, records_ptr, counts_ptr, next_ptr, done_ptr, a_ptr, rows_cap: int,
                   row_bytes: int, record_cap: int, groups: int) -> int:
        """Let the launch copy duplicate rows inside the packed A buffer itself (send-once
        exchange, ``bmoe_plan_set_expand``); ``records_ptr`` None switches it off."""
        return int(self._lib.bmoe_plan_set_expand(self._handle, records_ptr or None, counts_ptr,
                                                  next_ptr, done_ptr, a_ptr, rows_cap, row_bytes,
                                                  record_cap, groups))

    def set_push(self, origin_ptr, expert_row_ptr, y_bases_ptr, ranks: int, y_rows_cap: int) -> int:
        """Send result rows straight to their origin ranks' buffers instead of D (see
        ``bmoe_plan_set_push``); ``origin_ptr`` None switches back."""
        return int(self._lib.bmoe_plan_set_push(self._handle, origin_ptr, expert_row_ptr,
                                                y_bases_ptr, ranks, y_rows_cap))

    def poll(self) -> tuple[int, _capi.DeviceReport]:
        report = _capi.DeviceReport()
        status = int(self._lib.bmoe_plan_poll(self._handle, C.byref(report)))
        return status, report

    def stats(self) -> _capi.PlanStats:
        out = _capi.PlanStats()
        self._lib.bmoe_plan_stats_get(self._handle, C.byref(out))
        return out

    def worklist(self) -> np.ndarray:
        """The device worklist copied back to the host (structured array)."""
        total = self.stats().total_tiles
        tiles = (_capi.Tile * max(1, total))()
        count = C.c_uint32(0)
        _capi.check(
            self._lib.bmoe_plan_read_worklist(self._handle, tiles, total, C.byref(count)),
            "bmoe_plan_read_worklist",
        )
        return tiles_to_numpy(tiles, int(count.value))

    def set_observers(self, tile_visits=None, cta_tiles=None) -> int:
        self._observers = (tile_visits, cta_tiles)
        return int(self._lib.bmoe_plan_set_observers(
            self._handle,
            tile_visits.data_ptr() if tile_visits is not None else None,
            cta_tiles.data_ptr() if cta_tiles is not None else None,
        ))


    def set_trace(self, trace=None) -> int:
        """``trace``: CUDA int64 tensor [threadblock_count, 16] of wait-cycle counters."""
        self._trace = trace
        return int(self._lib.bmoe_plan_set_trace(
            self._handle, trace.data_ptr() if trace is not None else None))


def grouped_gemm(a, w, d, tokens_per_expert: Sequence[int], **options) -> None:
    """One-shot packed grouped GEMM on the current CUDA device; raises on error."""
    plan = GroupedGemmPlan()
    try:
        _capi.check(plan.initialize_packed(a, w, d, tokens_per_expert, **options),
                    "bmoe_plan_initialize")
        _capi.check(plan.run(options.get("stream")), "bmoe_plan_run")
        status, report = plan.poll()
        if status != _capi.OK:
            raise _capi.EngineError(status, f"grouped_gemm (site {report.code}, cta {report.cta})")
    finally:
        plan.close()


# ------------------------------------------------------- device worklist --


def worklist_layout(experts: int) -> _capi.WorklistLayout:
    out = _capi.WorklistLayout()
    _capi.check(_capi.load().bmoe_worklist_layout_for(experts, C.byref(out)),
                "bmoe_worklist_layout_for")
    return out


def build_worklist_on_device(counts_dev, n: int, tile_m: int, tile_n: int, *,
                             order: int = _capi.ORDER_EXPERT,
                             raster: int = _capi.RASTER_N_FASTEST,
                             tile_capacity: int, stream=None):
    """Runs the integer worklist kernels on ``counts_dev`` (CUDA int32 tensor).

    Returns ``(tiles, workspace, layout)``: ``tiles`` is a CUDA uint8 tensor of
    ``tile_capacity * 20`` bytes holding the records, ``workspace`` a CUDA uint8
    tensor whose regions ``layout`` describes. Nothing is synchronised.
    """
    import torch

    experts = int(counts_dev.numel())
    layout = worklist_layout(experts)
    device = counts_dev.device
    tiles = torch.empty(max(1, tile_capacity) * 20, dtype=torch.uint8, device=device)
    workspace = torch.empty(layout.bytes + 256, dtype=torch.uint8, device=device)
    base = (workspace.data_ptr() + 255) // 256 * 256
    request = _capi.WorklistRequest(experts=experts, n=n, tile_m=tile_m, tile_n=tile_n,
                                    order=order, raster=raster)
    _capi.check(
        _capi.load().bmoe_worklist_build(
            counts_dev.data_ptr(), C.byref(request), tiles.data_ptr(), tile_capacity,
            base, _stream_ptr(stream)),
        "bmoe_worklist_build",
    )
    offset = base - workspace.data_ptr()
    return tiles, workspace[offset:], layout


def read_worklist_arrays(workspace, layout: _capi.WorklistLayout, experts: int) -> dict:
    """Copies the builder's auxiliary arrays to the host as numpy arrays."""
    raw = workspace.cpu().numpy()

    def view(off: int, dtype: str, count: int) -> np.ndarray:
        width = np.dtype(dtype).itemsize
        return raw[off:off + width * count].view(dtype).copy()

    totals = view(layout.off_totals, "<u4", 8)
    return {
        "total_tiles": int(totals[0]),
        "active_experts": int(totals[1]),
        "total_rows": int(totals[2]) | (int(totals[3]) << 32),
        "total_valid_elements": int(totals[4]) | (int(totals[5]) << 32),
        "overflow": int(totals[6]),
        "row_offsets": view(layout.off_row_offsets, "<u8", experts + 1),
        "expert_m_tiles": view(layout.off_expert_m_tiles, "<u4", experts),
        "expert_tiles": view(layout.off_expert_tiles, "<u4", experts),
        "tile_offsets": view(layout.off_tile_offsets, "<u4", experts + 1),
        "active_ids": view(layout.off_active_ids, "<u4", experts),
        "visit_order": view(layout.off_visit_order, "<u4", experts),
        "visit_tile_offsets": view(layout.off_visit_tile_offsets, "<u4", experts + 1),
    }


# ----------------------------------------------------------------- probe --


def launch_scheduler_probe(scheduler: int, tiles_dev, tile_count: int, cta_count: int, *,
                           claim_size: int = 1, work_scale: int = 1, next_tile=None,
                           tile_visits=None, tile_checksums=None, cta_tile_counts=None,
                           cta_valid_elements=None, stream=None) -> int:
    """``launch_scheduler_probe`` of the reference; tensors are CUDA tensors."""

    def ptr(t):
        return t.data_ptr() if t is not None else None

    args = _capi.ProbeArgs(
        tiles=ptr(tiles_dev), tile_count=tile_count, cta_count=cta_count,
        claim_size=claim_size, work_scale=work_scale, next_tile=ptr(next_tile),
        tile_visits=ptr(tile_visits), tile_checksums=ptr(tile_checksums),
        cta_tile_counts=ptr(cta_tile_counts), cta_valid_elements=ptr(cta_valid_elements),
        stream=_stream_ptr(stream),
    )
    return int(_capi.load().bmoe_probe_launch(scheduler, C.byref(args)))
