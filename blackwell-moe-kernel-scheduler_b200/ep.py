"""Expert-parallel layer: experts sharded across ranks, tokens exchanged by
all-to-all, the local grouped GEMM run by the sm_100a engine.

The reference has no multi-GPU code (agent/search_space.yaml:10-13); this layer
adds the one exchange step the path needs. One process per GPU
(``torch.distributed``, NCCL over NVLink); the only collectives are a small
count all-gather and one all-to-all each side of the GEMM. Remote rows land in
local HBM through NCCL before any CTA touches them.

Per step and rank:
  1. count this rank's routed rows per expert, all-gather the counts
  2. gather token rows into send order (by owner rank, then expert id)
  3. all-to-all dispatch
  4. gather received rows (source-major) into the expert-major packed ``A``
  5. grouped GEMM over the local experts (any scheduling policy)
  6. inverse gather, all-to-all combine, inverse gather to assignment order

Placement is fixed per deployment (weights live on their owner):
``place_experts`` balances GEMM tiles per rank.
"""

from __future__ import annotations

import ctypes as C
from typing import Sequence

from . import _capi


def place_experts(global_counts: Sequence[int], ranks: int, n: int, *, tile_m: int = 128,
                  tile_n: int = 256, max_experts_per_rank: int = 0):
    """Expert -> owner rank by tile-count balance; returns (owner list, tiles per rank)."""
    experts = len(global_counts)
    counts = (C.c_uint32 * max(1, experts))(*[int(c) for c in global_counts])
    owner = (C.c_uint32 * max(1, experts))()
    loads = (C.c_uint64 * max(1, ranks))()
    _capi.check(
        _capi.load().bmoe_ep_place_experts(counts, experts, ranks, n, tile_m, tile_n,
                                           max_experts_per_rank, owner, loads),
        "bmoe_ep_place_experts")
    return [int(x) for x in owner][:experts], [int(x) for x in loads][:ranks]


def split_and_place_experts(global_counts: Sequence[int], ranks: int, n: int, *,
                            tile_m: int = 128, tile_n: int = 256, max_share: float = 0.5):
    """Placement with ROW SHARDS for hot experts. An expert whose tile count exceeds
    ``max_share`` of one rank's fair share (total tiles / ranks) is cut into that many
    shards of about equal rows (at most one per rank); every shard is then placed like
    an expert by ``place_experts``. The ranks that own shards of an expert each hold a
    copy of its weights; which shard a routed row goes to is decided per assignment
    (assignment index modulo the shard count), and no result row depends on it.

    Returns (parts, shard_owner, loads): ``parts[e]`` shards of expert e (1 = whole),
    shards numbered expert-major (shard id = sum(parts[:e]) + p), ``shard_owner[s]``
    the owning rank, ``loads`` the tiles per rank."""
    counts = [int(c) for c in global_counts]
    col_tiles = -(-n // tile_n)
    tiles = [-(-c // tile_m) * col_tiles for c in counts]
    fair = sum(tiles) / max(1, ranks)
    parts = []
    for t in tiles:
        want = 1 if ranks <= 1 or fair <= 0 else -(-t // max(1, int(max_share * fair)))
        parts.append(max(1, min(ranks, want)))
    shard_counts = []
    for c, p in zip(counts, parts):
        shard_counts.extend(c // p + (1 if q < c % p else 0) for q in range(p))
    shard_owner, loads = place_experts(shard_counts, ranks, n, tile_m=tile_m, tile_n=tile_n)
    return parts, shard_owner, loads


class CudaOps:
    """Device operations of the layer, all through the engine's C interface."""

    def __init__(self, scheduler="auto", **plan_options):
        from .engine import GroupedGemmPlan

        self._lib = _capi.load()
        self._plans = [GroupedGemmPlan()]
        self.scheduler = scheduler
        self.plan_options = plan_options
        self.launches = 0

    def gather_rows(self, src, index, out=None):
        import torch

        rows = int(index.numel())
        width = int(src.shape[1])
        if out is None:
            out = torch.empty(rows, width, dtype=src.dtype, device=src.device)
        if not src.is_cuda:
            raise RuntimeError("the engine has no CPU path: gather_rows needs CUDA tensors")
        stream = torch.cuda.current_stream().cuda_stream
        _capi.check(
            self._lib.bmoe_gather_rows(src.data_ptr(), out.data_ptr(), index.data_ptr(), rows,
                                       int(src.shape[0]), width * src.element_size(),
                                       stream or None),
            "bmoe_gather_rows")
        if rows:
            self.launches += 1
        return out

    def combine_topk(self, src, rows, weights=None, out=None):
        """out[t] = bf16(sum_j weights[t, j] * src[rows[t, j]]) in FP32, j ascending;
        ``rows`` [tokens, top_k] int64 (negative = dropped), ``weights`` float32 or None."""
        import torch

        if not src.is_cuda:
            raise RuntimeError("the engine has no CPU path: combine_topk needs CUDA tensors")
        tokens, top_k = int(rows.shape[0]), int(rows.shape[1])
        n = int(src.shape[1])
        if out is None:
            out = torch.empty(tokens, n, dtype=src.dtype, device=src.device)
        rows = rows.contiguous()
        if weights is not None:
            weights = weights.to(torch.float32).contiguous()
        base = torch.tensor([src.data_ptr()], dtype=torch.int64, device=src.device)
        _capi.check(
            self._lib.bmoe_combine_topk(base.data_ptr(), 1, int(src.shape[0]), None,
                                        rows.data_ptr(),
                                        weights.data_ptr() if weights is not None else None,
                                        tokens, top_k, n, out.data_ptr(), 0,
                                        torch.cuda.current_stream().cuda_stream or None),
            "bmoe_combine_topk")
        if tokens:
            self.launches += 1
        return out

    def grouped_gemm(self, a, w, counts, out=None, slot=0):
        """``slot`` selects the plan object; launches that may be in flight at the
        same time (pipelined expert groups) must use different slots."""
        import torch

        from .engine import GroupedGemmPlan

        while len(self._plans) <= slot:
            self._plans.append(GroupedGemmPlan())
        plan = self._plans[slot]
        total = int(sum(counts))
        n = int(w.shape[1])
        if out is None:
            out = torch.empty(total, n, dtype=a.dtype, device=a.device)
        if total == 0:
            return out
        stream = torch.cuda.current_stream()
        _capi.check(plan.initialize_packed(a, w, out, counts, scheduler=self.scheduler,
                                           stream=stream, **self.plan_options),
                    "bmoe_plan_initialize")
        _capi.check(plan.run(stream), "bmoe_plan_run")
        self.launches += 3  # worklist plan + expand, grouped GEMM
        return out

    def poll(self):
        for plan in self._plans:
            status, report = plan.poll()
            if status not in (_capi.OK, _capi.INVALID_ARGUMENT):  # INVALID = never initialised
                raise _capi.EngineError(
                    status, f"grouped GEMM (site {report.code}, cta {report.cta})")


class ExpertParallelLayer:
    """One expert-parallel grouped GEMM (e.g. an MoE up-projection)."""

    def __init__(self, owner: Sequence[int], n: int, k: int, *, rank: int, world: int,
                 group=None, ops=None, pipeline_groups: int = 1):
        """``pipeline_groups`` > 1 splits every rank's experts into that many
        groups and overlaps the exchange of one group with the GEMM of another."""
        self.pipeline_groups = max(1, int(pipeline_groups))
        self.owner = [int(o) for o in owner]
        self.experts = len(self.owner)
        self.n, self.k = n, k
        self.rank, self.world = rank, world
        self.group = group
        self.ops = ops if ops is not None else CudaOps()
        # Experts in send order: by owner rank, then expert id.
        self.send_order = sorted(range(self.experts), key=lambda e: (self.owner[e], e))
        self.local_experts = [e for e in range(self.experts) if self.owner[e] == rank]
        self.timings = {}

    def _host_tables(self):
        import torch

        if not hasattr(self, "_tables"):
            owner_t = torch.tensor(self.owner, dtype=torch.int64)
            local_t = torch.tensor(self.local_experts, dtype=torch.int64)
            position = torch.empty(self.experts, dtype=torch.int64)
            position[torch.tensor(self.send_order, dtype=torch.int64)] = torch.arange(self.experts)
            self._tables = (owner_t, local_t, position)
        return self._tables

    def _position_on(self, dev):
        if getattr(self, "_position_dev", None) is None or self._position_dev.device != dev:
            self._position_dev = self._host_tables()[2].to(dev)
        return self._position_dev

    # -- collectives (skipped when there is a single rank) --
    def _all_gather_counts(self, local_counts):
        import torch
        import torch.distributed as dist

        if self.world == 1:
            return local_counts.reshape(1, -1)
        flat = torch.empty(self.world * self.experts, dtype=local_counts.dtype,
                           device=local_counts.device)
        dist.all_gather_into_tensor(flat, local_counts, group=self.group)
        return flat.reshape(self.world, self.experts)

    def _all_to_all(self, send, send_splits, recv_splits):
        import torch
        import torch.distributed as dist

        if self.world == 1:
            return send
        recv = torch.empty(sum(recv_splits), send.shape[1], dtype=send.dtype, device=send.device)
        dist.all_to_all_single(recv, send, recv_splits, send_splits, group=self.group)
        return recv

    def forward(self, x, expert_ids, w_local, record_events=False, topk_weights=None):
        """x [T_local, k]; expert_ids [T_local, top_k] int64 (device of x);
        w_local [len(local_experts), n, k] in ascending expert id.
        Returns y [T_local * top_k, n]: row j is token j // top_k routed to
        expert_ids.flatten()[j]. With ``topk_weights`` [T_local, top_k] (float32) the
        last step is the weighted top-k sum instead and y is [T_local, n]."""
        import torch

        if self.world > 1 and self.pipeline_groups > 1:
            if topk_weights is not None:
                raise ValueError("topk_weights is not supported with pipeline_groups > 1")
            return self._forward_pipelined(x, expert_ids, w_local, record_events)

        dev = x.device
        top_k = int(expert_ids.shape[1])
        flat_ids = expert_ids.reshape(-1)
        assignments = int(flat_ids.numel())
        marks = []

        def mark(name):
            if record_events and x.is_cuda:
                ev = torch.cuda.Event(enable_timing=True)
                ev.record(torch.cuda.current_stream())
                marks.append((name, ev))

        mark("start")
        # 1. counts
        # scatter_add instead of bincount: no device synchronisation to size the output
        local_counts = torch.zeros(self.experts, dtype=torch.int64, device=dev)
        local_counts.scatter_add_(0, flat_ids, torch.ones_like(flat_ids))
        counts_all = self._all_gather_counts(local_counts).cpu()  # [world, experts], host
        owner_t, local_t, position = self._host_tables()
        send_splits = torch.zeros(self.world, dtype=torch.int64).scatter_add_(
            0, owner_t, counts_all[self.rank]).tolist()
        recv_matrix = counts_all[:, local_t]                        # [world, E_local]
        recv_splits = recv_matrix.sum(dim=1).tolist()
        local_m = recv_matrix.sum(dim=0).tolist()
        mark("counts")

        # 2. send order: stable sort of the assignments by position of their expert
        keys = self._position_on(dev)[flat_ids]
        perm = torch.sort(keys, stable=True).indices               # assignment ids in send order
        send = self.ops.gather_rows(x, torch.div(perm, top_k, rounding_mode="floor"))
        mark("pack")

        # 3. dispatch
        recv = self._all_to_all(send, send_splits, recv_splits)
        mark("dispatch")

        total_local = int(sum(local_m))
        if self.world == 1:
            # A single rank receives its own send buffer, which is already
            # expert-major: nothing to re-pack in either direction.
            d_packed = self.ops.grouped_gemm(recv, w_local, local_m)
            mark("gemm")
            inv_perm = torch.empty(assignments, dtype=torch.int64, device=dev)
            inv_perm[perm] = torch.arange(assignments, device=dev, dtype=torch.int64)
            y = self._finish(d_packed, inv_perm, top_k, topk_weights)
            mark("finish")
            self._marks = marks
            self.last_local_m = local_m
            return y

        # 4. source-major -> expert-major. Segment (e, s) of the packed A starts at
        # recv_offset[s] + prefix of source s over local experts before e.
        seg_len = recv_matrix.t().contiguous().reshape(-1)          # (e, s) order
        src_base = torch.cumsum(torch.tensor([0] + recv_splits[:-1], dtype=torch.int64), 0)
        within = torch.cumsum(recv_matrix, dim=1) - recv_matrix      # [world, E_local]
        seg_start = (src_base[:, None] + within).t().contiguous().reshape(-1)
        seg_len_d, seg_start_d = seg_len.to(dev), seg_start.to(dev)
        out_start = torch.cumsum(seg_len_d, 0) - seg_len_d
        index = (torch.repeat_interleave(seg_start_d - out_start, seg_len_d,
                                         output_size=total_local)
                 + torch.arange(total_local, device=dev, dtype=torch.int64))
        a_packed = self.ops.gather_rows(recv, index)
        mark("unpack")

        # 5. local grouped GEMM
        d_packed = self.ops.grouped_gemm(a_packed, w_local, local_m)
        mark("gemm")

        # 6. back: expert-major -> source-major, combine, -> assignment order
        inverse = torch.empty(total_local, dtype=torch.int64, device=dev)
        inverse[index] = torch.arange(total_local, device=dev, dtype=torch.int64)
        d_send = self.ops.gather_rows(d_packed, inverse)
        mark("repack")
        d_recv = self._all_to_all(d_send, recv_splits, send_splits)
        mark("combine")
        inv_perm = torch.empty(assignments, dtype=torch.int64, device=dev)
        inv_perm[perm] = torch.arange(assignments, device=dev, dtype=torch.int64)
        y = self._finish(d_recv, inv_perm, top_k, topk_weights)
        mark("finish")
        self._marks = marks
        self.last_local_m = local_m
        return y

    def _finish(self, rows_in_send_order, inv_perm, top_k, topk_weights):
        """Assignment order (plain gather) or, with weights, the weighted top-k sum:
        one kernel either way."""
        if topk_weights is None:
            return self.ops.gather_rows(rows_in_send_order, inv_perm)
        return self.ops.combine_topk(rows_in_send_order, inv_perm.reshape(-1, top_k),
                                     topk_weights)

    # ------------------------------------------------------------ pipelined --
    def _group_tables(self):
        """Expert -> pipeline group, and the send order (group, owner, expert)."""
        import torch

        if not hasattr(self, "_gtables"):
            groups = self.pipeline_groups
            group_of = [0] * self.experts
            local_bounds = None
            for r in range(self.world):
                mine = [e for e in range(self.experts) if self.owner[e] == r]
                for i, e in enumerate(mine):
                    group_of[e] = i * groups // max(1, len(mine))
                if r == self.rank:
                    cuts = [0] * (groups + 1)
                    for i in range(len(mine)):
                        cuts[i * groups // max(1, len(mine)) + 1] = i + 1
                    for g in range(1, groups + 1):
                        cuts[g] = max(cuts[g], cuts[g - 1])
                    local_bounds = cuts
            order = sorted(range(self.experts), key=lambda e: (group_of[e], self.owner[e], e))
            position = torch.empty(self.experts, dtype=torch.int64)
            position[torch.tensor(order, dtype=torch.int64)] = torch.arange(self.experts)
            self._gtables = (torch.tensor(group_of, dtype=torch.int64), position, local_bounds)
        return self._gtables

    def _forward_pipelined(self, x, expert_ids, w_local, record_events=False):
        """Same result as forward(); the experts of every rank are split into
        ``pipeline_groups`` groups whose dispatch / GEMM / combine overlap: all
        dispatches are queued on the communication stream up front, each group's
        GEMM starts when its rows have arrived, and its combine is queued behind."""
        import torch
        import torch.distributed as dist

        dev = x.device
        groups = self.pipeline_groups
        top_k = int(expert_ids.shape[1])
        flat_ids = expert_ids.reshape(-1)
        assignments = int(flat_ids.numel())
        marks = []

        def mark(name):
            if record_events and x.is_cuda:
                ev = torch.cuda.Event(enable_timing=True)
                ev.record(torch.cuda.current_stream())
                marks.append((name, ev))

        mark("start")
        local_counts = torch.zeros(self.experts, dtype=torch.int64, device=dev)
        local_counts.scatter_add_(0, flat_ids, torch.ones_like(flat_ids))
        counts_all = self._all_gather_counts(local_counts).cpu()
        owner_t, local_t, _ = self._host_tables()
        group_t, position, bounds = self._group_tables()
        send_matrix = torch.zeros(groups * self.world, dtype=torch.int64).scatter_add_(
            0, group_t * self.world + owner_t, counts_all[self.rank]).reshape(groups, self.world)
        send_rows = send_matrix.sum(dim=1).tolist()
        send_off = [0]
        for r in send_rows:
            send_off.append(send_off[-1] + r)
        mark("counts")

        if getattr(self, "_gposition_dev", None) is None or self._gposition_dev.device != dev:
            self._gposition_dev = position.to(dev)
        keys = self._gposition_dev[flat_ids]
        perm = torch.sort(keys, stable=True).indices
        token_of = torch.div(perm, top_k, rounding_mode="floor")
        d_recv = torch.empty(assignments, self.n, dtype=x.dtype, device=dev)

        # queue every group's pack + dispatch
        staged = []
        for g in range(groups):
            lo, hi = bounds[g], bounds[g + 1]
            recv_matrix = counts_all[:, local_t[lo:hi]]                 # [world, E_g]
            recv_splits = recv_matrix.sum(dim=1).tolist()
            send_splits = send_matrix[g].tolist()
            send = self.ops.gather_rows(x, token_of[send_off[g]:send_off[g + 1]])
            recv = torch.empty(sum(recv_splits), self.k, dtype=x.dtype, device=dev)
            work = dist.all_to_all_single(recv, send, recv_splits, send_splits,
                                          group=self.group, async_op=True)
            staged.append((lo, hi, recv_matrix, recv_splits, send_splits, send, recv, work))
        mark("pack+dispatch issue")

        combines = []
        local_m_all = []
        for g, (lo, hi, recv_matrix, recv_splits, send_splits, send, recv, work) in enumerate(staged):
            work.wait()
            mark(f"dispatch {g} arrived")
            local_m = recv_matrix.sum(dim=0).tolist()
            local_m_all.extend(local_m)
            total_local = int(sum(local_m))
            seg_len = recv_matrix.t().contiguous().reshape(-1)
            src_base = torch.cumsum(torch.tensor([0] + recv_splits[:-1], dtype=torch.int64), 0)
            within = torch.cumsum(recv_matrix, dim=1) - recv_matrix
            seg_start = (src_base[:, None] + within).t().contiguous().reshape(-1)
            seg_len_d, seg_start_d = seg_len.to(dev), seg_start.to(dev)
            out_start = torch.cumsum(seg_len_d, 0) - seg_len_d
            index = (torch.repeat_interleave(seg_start_d - out_start, seg_len_d,
                                             output_size=total_local)
                     + torch.arange(total_local, device=dev, dtype=torch.int64))
            a_packed = self.ops.gather_rows(recv, index)
            d_packed = self.ops.grouped_gemm(a_packed, w_local[lo:hi], local_m, slot=g)
            inverse = torch.empty(total_local, dtype=torch.int64, device=dev)
            inverse[index] = torch.arange(total_local, device=dev, dtype=torch.int64)
            d_send = self.ops.gather_rows(d_packed, inverse)
            back = d_recv[send_off[g]:send_off[g + 1]]
            cwork = dist.all_to_all_single(back, d_send, send_splits, recv_splits,
                                           group=self.group, async_op=True)
            combines.append((cwork, d_send, a_packed, d_packed))
            mark(f"gemm {g}")
        for cwork, *_ in combines:
            cwork.wait()
        mark("combine")
        inv_perm = torch.empty(assignments, dtype=torch.int64, device=dev)
        inv_perm[perm] = torch.arange(assignments, device=dev, dtype=torch.int64)
        y = self.ops.gather_rows(d_recv, inv_perm)
        mark("finish")
        self._marks = marks
        self.last_local_m = local_m_all
        return y

    def phase_times_ms(self):
        """Per-phase device times of the last forward(record_events=True)."""
        import torch

        torch.cuda.synchronize()
        out = {}
        for (_, a), (name, b) in zip(self._marks[:-1], self._marks[1:]):
            out[name] = a.elapsed_time(b)
        return out
