"""Expert-parallel layer with the exchange fused into two routing kernels over
peer memory (NVLink), instead of NCCL all-to-all plus local re-packing.

Per step and rank:
  1. count routed rows per expert, all-gather the counts (NCCL, tiny)
  2. ONE kernel pushes every token row straight into its owner's expert-major
     packed ``A`` (peer stores over NVLink); the destination row of each
     assignment follows from the count matrix, so no intermediate send / receive
     buffers and no re-packing exist
  3. stream-ordered barrier (one-element all-reduce), local grouped GEMM into a
     peer-readable ``D``, barrier
  4. ONE kernel pulls each assignment's result row from its owner's ``D`` back
     into assignment order (peer loads)

The buffers are plain device allocations shared through CUDA IPC
(``bmoe_peer_alloc`` / ``bmoe_peer_open``); CTAs of the GEMM only ever TMA from
local memory. ``ep.ExpertParallelLayer`` (NCCL all-to-all) computes the same
result and stays available as the baseline exchange.
"""

from __future__ import annotations

import ctypes as C
from typing import Sequence

from . import _capi


class _RawCudaBuffer:
    """Wraps a raw device pointer for ``torch.as_tensor`` (CUDA array interface)."""

    def __init__(self, ptr: int, elements: int):
        self.__cuda_array_interface__ = {
            "shape": (elements,), "typestr": "<i2", "data": (ptr, False), "version": 2,
        }


class RoutePlanner:
    """Destination of every local assignment in its owner's expert-major buffer.

    Static per (owner map, rank): the tables below. Per step, ``plan`` needs the
    host count matrix [world, experts] and the device expert ids.

    Rows of one expert are laid out by source rank, then by assignment order -
    the order of a single-GPU run. The traversal order of the returned arrays is
    staggered by rank (rank r starts with the rows bound for rank r+1, then r+2,
    ...), so that at any moment the ranks push to, or pull from, different GPUs
    instead of all converging on the owner of the busiest expert.
    """

    def __init__(self, owner: Sequence[int], rank: int, world: int):
        import torch

        self.rank, self.world = rank, world
        self.experts = len(owner)
        self.owner_t = torch.tensor(list(owner), dtype=torch.int64)
        # experts ordered by (owner, id): packed order inside every owner's buffer
        self.by_owner = torch.tensor(
            sorted(range(self.experts), key=lambda e: (owner[e], e)), dtype=torch.int64)
        self.owner_in_order = self.owner_t[self.by_owner]
        # traversal order of this rank: staggered destination, then expert id
        stagger = (self.owner_t - rank - 1) % world
        self.key_of_expert = stagger * self.experts + torch.arange(self.experts)
        self.by_key = torch.argsort(self.key_of_expert)
        self._dev = None

    def _device_tables(self, dev):
        if self._dev is None or self._dev[0].device != dev:
            self._dev = (self.key_of_expert.to(dev), self.owner_t.to(dev).to(self._i32()))
        return self._dev

    @staticmethod
    def _i32():
        import torch

        return torch.int32

    def plan(self, counts_all, flat_ids, top_k: int):
        """Returns (perm, src_token, dst_rank, dst_row); ``perm[i]`` is the local
        assignment handled i-th, bound for row ``dst_row[i]`` of rank ``dst_rank[i]``."""
        import torch

        dev = flat_ids.device
        totals = counts_all.sum(dim=0)
        # offset of each expert inside its owner's buffer
        t_order = totals[self.by_owner]
        excl = torch.cumsum(t_order, 0) - t_order
        per_owner = torch.zeros(self.world, dtype=torch.int64).scatter_add_(
            0, self.owner_in_order, t_order)
        seg_base = torch.cumsum(per_owner, 0) - per_owner
        owner_off = torch.empty(self.experts, dtype=torch.int64)
        owner_off[self.by_owner] = excl - seg_base[self.owner_in_order]
        dst_base = owner_off + counts_all[:self.rank].sum(dim=0)
        # first position of each expert in this rank's traversal order
        local = counts_all[self.rank]
        l_order = local[self.by_key]
        start = torch.empty(self.experts, dtype=torch.int64)
        start[self.by_key] = torch.cumsum(l_order, 0) - l_order
        tables = torch.stack([dst_base, start]).to(dev)               # one small H2D copy

        key_dev, owner_dev = self._device_tables(dev)
        perm = torch.sort(key_dev[flat_ids], stable=True).indices
        sorted_e = flat_ids[perm]
        within = torch.arange(perm.numel(), device=dev, dtype=torch.int64) - tables[1][sorted_e]
        dst_row = tables[0][sorted_e] + within
        dst_rank = owner_dev[sorted_e]
        src_token = torch.div(perm, top_k, rounding_mode="floor")
        return perm, src_token, dst_rank, dst_row


def plan_routes(counts_all, owner: Sequence[int], rank: int, flat_ids, top_k: int):
    """One-shot form of ``RoutePlanner(...).plan(...)``."""
    return RoutePlanner(owner, rank, counts_all.shape[0]).plan(counts_all, flat_ids, top_k)


class PeerBuffers:
    """``A`` [rows_cap, k] and ``D`` [rows_cap, n] BF16 on every rank, each mapped by
    all ranks of the node."""

    def __init__(self, rows_cap: int, k: int, n: int, *, rank: int, world: int, group=None):
        import torch
        import torch.distributed as dist

        self._lib = _capi.load()
        self.rows_cap, self.k, self.n, self.rank, self.world = rows_cap, k, n, rank, world
        dev = torch.device("cuda", torch.cuda.current_device())
        self._own = []
        handles = torch.zeros(2, 64, dtype=torch.uint8)
        ptrs = []
        for i, width in enumerate((k, n)):
            ptr = C.c_void_p()
            buf = (C.c_uint8 * 64)()
            _capi.check(self._lib.bmoe_peer_alloc(rows_cap * width * 2, C.byref(ptr), buf),
                        "bmoe_peer_alloc")
            self._own.append(ptr.value)
            handles[i] = torch.tensor(list(buf), dtype=torch.uint8)
            ptrs.append(ptr.value)
        self.a = torch.as_tensor(_RawCudaBuffer(ptrs[0], rows_cap * k), device=dev) \
            .view(torch.bfloat16).view(rows_cap, k)
        self.d = torch.as_tensor(_RawCudaBuffer(ptrs[1], rows_cap * n), device=dev) \
            .view(torch.bfloat16).view(rows_cap, n)
        self._opened = []
        a_bases, d_bases = [0] * world, [0] * world
        a_bases[rank], d_bases[rank] = ptrs[0], ptrs[1]
        if world > 1:
            gathered = torch.zeros(world, 2, 64, dtype=torch.uint8, device=dev)
            dist.all_gather_into_tensor(gathered.view(-1), handles.to(dev).view(-1), group=group)
            gathered = gathered.cpu()
            for r in range(world):
                if r == rank:
                    continue
                for i, table in enumerate((a_bases, d_bases)):
                    raw = (C.c_uint8 * 64)(*gathered[r, i].tolist())
                    ptr = C.c_void_p()
                    _capi.check(self._lib.bmoe_peer_open(raw, C.byref(ptr)), "bmoe_peer_open")
                    self._opened.append(ptr.value)
                    table[r] = ptr.value
        self.a_bases = torch.tensor(a_bases, dtype=torch.int64, device=dev)
        self.d_bases = torch.tensor(d_bases, dtype=torch.int64, device=dev)

    def close(self):
        import torch

        torch.cuda.synchronize()
        for p in self._opened:
            self._lib.bmoe_peer_close(p)
        self._opened = []
        self.a = self.d = None
        for p in self._own:
            self._lib.bmoe_peer_free(p)
        self._own = []


class PeerExpertParallelLayer:
    """Same interface and result as ``ep.ExpertParallelLayer``; exchange by two
    routing kernels over peer memory."""

    def __init__(self, owner: Sequence[int], n: int, k: int, *, rank: int, world: int,
                 rows_cap: int, group=None, scheduler="dynamic_queue", route_ctas: int = 0,
                 **plan_options):
        import torch

        from .engine import GroupedGemmPlan

        self._lib = _capi.load()
        self.owner = [int(o) for o in owner]
        self.experts = len(self.owner)
        self.n, self.k, self.rank, self.world, self.group = n, k, rank, world, group
        self.local_experts = [e for e in range(self.experts) if self.owner[e] == rank]
        self.buffers = PeerBuffers(rows_cap, k, n, rank=rank, world=world, group=group)
        self.plan = GroupedGemmPlan()
        self.scheduler, self.plan_options = scheduler, plan_options
        self.route_ctas = route_ctas
        self.launches = 0
        dev = torch.device("cuda", torch.cuda.current_device())
        self._token = torch.zeros(1, dtype=torch.int32, device=dev)
        self._local_t = torch.tensor(self.local_experts, dtype=torch.int64)
        self._planner = RoutePlanner(self.owner, rank, world)
        self._base_cache = {}

    def close(self):
        self.plan.close()
        self.buffers.close()

    def _base_of(self, tensor):
        """One-entry device pointer table for a local tensor (cached by address)."""
        import torch

        key = tensor.data_ptr()
        if key not in self._base_cache:
            if len(self._base_cache) > 64:
                self._base_cache.clear()
            self._base_cache[key] = torch.tensor([key], dtype=torch.int64, device=tensor.device)
        return self._base_cache[key]

    def _barrier(self):
        """Stream-ordered cross-rank barrier (no host synchronisation)."""
        import torch.distributed as dist

        if self.world > 1:
            dist.all_reduce(self._token, group=self.group)

    def _route(self, src_bases, n_src, src_cap, src_rank, src_row, dst_bases, n_dst, dst_cap,
               dst_rank, dst_row, rows, row_bytes):
        import torch

        def ptr(t):
            return t.data_ptr() if t is not None else None

        _capi.check(
            self._lib.bmoe_route_rows(ptr(src_bases), n_src, src_cap, ptr(src_rank), ptr(src_row),
                                      ptr(dst_bases), n_dst, dst_cap, ptr(dst_rank), ptr(dst_row),
                                      rows, row_bytes, self.route_ctas,
                                      torch.cuda.current_stream().cuda_stream or None),
            "bmoe_route_rows")
        if rows:
            self.launches += 1

    def forward(self, x, expert_ids, w_local, record_events=False, topk_weights=None):
        """As ``ep.ExpertParallelLayer.forward``. With ``topk_weights`` the combine
        kernel reads every result row from its owner's memory and reduces the
        top_k rows of a token on the fly (y is [T_local, n])."""
        import torch
        import torch.distributed as dist

        dev = x.device
        top_k = int(expert_ids.shape[1])
        flat_ids = expert_ids.reshape(-1)
        assignments = int(flat_ids.numel())
        marks = []

        def mark(name):
            if record_events:
                ev = torch.cuda.Event(enable_timing=True)
                ev.record(torch.cuda.current_stream())
                marks.append((name, ev))

        mark("start")
        local_counts = torch.zeros(self.experts, dtype=torch.int64, device=dev)
        local_counts.scatter_add_(0, flat_ids, torch.ones_like(flat_ids))
        if self.world > 1:
            flat = torch.empty(self.world * self.experts, dtype=torch.int64, device=dev)
            dist.all_gather_into_tensor(flat, local_counts, group=self.group)
            counts_all = flat.reshape(self.world, self.experts).cpu()
        else:
            counts_all = local_counts.reshape(1, -1).cpu()
        local_m = counts_all[:, self._local_t].sum(dim=0).tolist()
        total_local = int(sum(local_m))
        if total_local > self.buffers.rows_cap:
            raise RuntimeError("routed rows exceed the peer buffer capacity")
        perm, src_token, dst_rank, dst_row = self._planner.plan(counts_all, flat_ids, top_k)
        mark("counts")

        # dispatch: push token rows into the owners' expert-major A
        x_base = self._base_of(x)
        self._route(x_base, 1, int(x.shape[0]), None, src_token,
                    self.buffers.a_bases, self.world, self.buffers.rows_cap, dst_rank, dst_row,
                    assignments, self.k * 2)
        self._barrier()
        mark("dispatch")

        stream = torch.cuda.current_stream()
        if total_local:
            _capi.check(self.plan.initialize_packed(self.buffers.a, w_local, self.buffers.d,
                                                    local_m, scheduler=self.scheduler,
                                                    stream=stream, **self.plan_options),
                        "bmoe_plan_initialize")
            _capi.check(self.plan.run(stream), "bmoe_plan_run")
            self.launches += 3
        self._barrier()
        mark("gemm")

        if topk_weights is not None:
            # combine + weighted reduction in one pass over peer memory
            by_rank = torch.empty(assignments, dtype=torch.int32, device=dev)
            by_row = torch.empty(assignments, dtype=torch.int64, device=dev)
            by_rank[perm] = dst_rank
            by_row[perm] = dst_row
            weights = topk_weights.to(torch.float32).contiguous()
            y = torch.empty(assignments // top_k, self.n, dtype=x.dtype, device=dev)
            _capi.check(
                self._lib.bmoe_combine_topk(self.buffers.d_bases.data_ptr(), self.world,
                                            self.buffers.rows_cap, by_rank.data_ptr(),
                                            by_row.data_ptr(), weights.data_ptr(),
                                            assignments // top_k, top_k, self.n, y.data_ptr(),
                                            self.route_ctas,
                                            torch.cuda.current_stream().cuda_stream or None),
                "bmoe_combine_topk")
            self.launches += 1
            # No barrier here: an owner rewrites D only after the barrier that follows
            # the NEXT dispatch, which every rank enters after this kernel.
            mark("combine")
            self._marks = marks
            self.last_local_m = local_m
            return y

        # combine: pull result rows back into assignment order
        y = torch.empty(assignments, self.n, dtype=x.dtype, device=dev)
        y_base = self._base_of(y)
        self._route(self.buffers.d_bases, self.world, self.buffers.rows_cap, dst_rank, dst_row,
                    y_base, 1, assignments, None, perm, assignments, self.n * 2)
        mark("combine")
        self._marks = marks
        self.last_local_m = local_m
        return y

    def poll(self):
        status, report = self.plan.poll()
        if status not in (_capi.OK, _capi.INVALID_ARGUMENT):
            raise _capi.EngineError(status, f"grouped GEMM (site {report.code}, cta {report.cta})")

    def phase_times_ms(self):
        import torch

        torch.cuda.synchronize()
        return {name: a.elapsed_time(b)
                for (_, a), (name, b) in zip(self._marks[:-1], self._marks[1:])}
