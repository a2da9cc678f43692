"""Expert-parallel layer whose exchange overlaps the grouped GEMM.

Same interface and result as ``ep.ExpertParallelLayer`` (NCCL all-to-all) and
``ep_peer.PeerExpertParallelLayer`` (two routing kernels with barriers). Here the
transfer and the math run at the same time:

* a dispatch kernel on a side stream pushes the rows bound for other GPUs into the
  owners' packed ``A`` group by group (experts are split into a few groups in
  packed order) and raises a flag per (group, source) on every peer;
* the grouped GEMM starts at once: its tile scheduler publishes the tiles of a
  group only when the flags of all other sources for that group are in, so early
  groups compute while late groups are still in flight;
* the epilogue of the GEMM writes every result row straight into the result buffer
  of the rank the row came from (the dispatcher leaves an origin record beside each
  row), so the way back is spread over the run time of the GEMM as well; a last
  small launch raises a "done" flag on every peer and the step ends when the other
  ranks' "done" flags are in. (``push_results=False`` keeps D local and sends the
  rows back with a separate kernel after the GEMM.)

Optionally (``copy_engine_min_bytes``) large (expert, source) blocks do not go through
the SMs: the source packs the rows of such a block into a local staging buffer in the
order they take in the owner's ``A`` and sends the block as ONE peer copy, followed in
the same stream by a 4-byte copy that raises a flag of a second plane; the gate of the
GEMM waits for both planes. Off by default (it measured slower than SM stores).

The only NCCL call per step is the all-gather of the per-expert counts. Kernels
of one GPU never wait on each other: rows that stay on the rank are copied by a
launch that precedes the GEMM in the same stream, and the gate looks at the flags
of other ranks only. Every device-side wait is bounded; ``poll()`` reports a wait
that ran out.
"""

from __future__ import annotations

import ctypes as C
from typing import Sequence

import numpy as np

from . import _capi


class StepPlanner:
    """Host tables of one step, vectorised; everything that depends only on the
    expert -> rank map is prepared once.

    Packed order on an owner: its experts in ascending id, and inside an expert the
    sources in ascending rank. Groups are contiguous runs of an owner's experts with
    about equal numbers of ``tile_m``-row tiles.
    """

    def __init__(self, owner: Sequence[int], rank: int, world: int, groups: int, tile_m: int = 256):
        self.rank, self.world, self.groups, self.tile_m = rank, world, max(1, groups), tile_m
        owner_a = np.asarray(list(owner), dtype=np.int64)
        self.experts = owner_a.size
        self.order = np.lexsort((np.arange(self.experts), owner_a))     # by (owner, id)
        self.owner_sorted = owner_a[self.order]
        # position in `order` where each expert's owner segment starts
        first = np.searchsorted(self.owner_sorted, np.arange(world), side="left")
        self.seg_start = first[self.owner_sorted]
        self.local = np.nonzero(owner_a == rank)[0]
        self.owner_a = owner_a

    def step(self, counts_all, copy_min_rows: int = 0):
        """``counts_all`` [world, experts] (numpy int64, identical on every rank). Returns a
        dict with ``local_experts``, ``local_m`` (rows per local expert), ``row_base``
        (int64 [experts]: first row of (expert, this rank) in the owner's A), ``group_of``
        (uint8 [experts]), ``group_local`` (uint8 per local expert), ``bucket_offset``
        (uint32 [groups + 3]: this rank's route entries per exchange group, then the rows
        that stay, then the rows of copy-engine blocks) and ``total_local``.

        ``copy_min_rows`` > 0: an (expert, source) block of at least that many rows whose
        owner is another rank travels as one peer copy. ``staging_row_base`` (int64
        [experts], -1 = not such a block) places this rank's blocks in its staging buffer,
        ``copy_experts`` lists them in sending order (group, owner, id) and ``copy_mask``
        (uint32 [groups]) has bit r set where source r sends such a block for one of this
        rank's experts of that group. Every rank derives the same decisions from the same
        count matrix."""
        counts_all = np.asarray(counts_all, dtype=np.int64)
        totals = counts_all.sum(axis=0)
        before_me = counts_all[:self.rank].sum(axis=0)
        t = totals[self.order]
        excl = np.cumsum(t) - t
        row_base = np.empty(self.experts, dtype=np.int64)
        row_base[self.order] = excl - excl[self.seg_start] + before_me[self.order]
        group_of = np.zeros(self.experts, dtype=np.uint8)
        if self.groups > 1:
            tiles = (t + self.tile_m - 1) // self.tile_m
            tiles_excl = np.cumsum(tiles) - tiles
            before = tiles_excl - tiles_excl[self.seg_start]
            per_owner = np.bincount(self.owner_sorted, weights=tiles, minlength=self.world)
            total = np.maximum(1, per_owner[self.owner_sorted].astype(np.int64))
            group_of[self.order] = np.minimum(self.groups - 1, before * self.groups // total)
        # entries this rank routes per bucket: exchange groups 0..G-1 (rows bound for other
        # ranks), then the rows that stay
        mine = counts_all[self.rank]
        away = self.owner_a != self.rank
        by_copy = away & (mine >= copy_min_rows) if copy_min_rows > 0 else np.zeros_like(away)
        by_sm = away & ~by_copy
        sizes = np.zeros(self.groups + 2, dtype=np.int64)
        sizes[:self.groups] = np.bincount(group_of[by_sm], weights=mine[by_sm],
                                          minlength=self.groups)[:self.groups]
        sizes[self.groups] = mine[~away].sum()
        sizes[self.groups + 1] = mine[by_copy].sum()
        bucket_offset = np.zeros(self.groups + 3, dtype=np.uint32)
        bucket_offset[1:] = np.cumsum(sizes)
        staging_row_base = np.full(self.experts, -1, dtype=np.int64)
        copy_experts = np.nonzero(by_copy)[0]
        if copy_experts.size:
            copy_experts = copy_experts[np.lexsort((copy_experts, self.owner_a[copy_experts],
                                                    group_of[copy_experts]))]
            rows = mine[copy_experts]
            staging_row_base[copy_experts] = np.cumsum(rows) - rows
        copy_mask = np.zeros(self.groups, dtype=np.uint32)
        if copy_min_rows > 0 and self.local.size:
            arrives = counts_all[:, self.local] >= copy_min_rows          # [world, local experts]
            arrives[self.rank] = False
            groups_local = group_of[self.local]
            for r in np.nonzero(arrives.any(axis=1))[0]:
                for g in np.unique(groups_local[arrives[r]]):
                    copy_mask[g] |= np.uint32(1 << int(r))
        local_m = totals[self.local]
        return {
            "local_experts": self.local.tolist(),
            "local_m": local_m,
            "row_base": row_base,
            "group_of": group_of,
            "group_local": group_of[self.local],
            "bucket_offset": bucket_offset,
            "total_local": int(local_m.sum()),
            "staging_row_base": staging_row_base,
            "copy_experts": copy_experts,
            "copy_mask": copy_mask,
        }


def plan_step(counts_all, owner: Sequence[int], rank: int, groups: int, tile_m: int = 256,
              copy_min_rows: int = 0):
    """One-shot form of ``StepPlanner(...).step(counts_all)`` with ``local_m`` as a list."""
    counts_all = np.asarray(counts_all, dtype=np.int64)
    out = StepPlanner(owner, rank, counts_all.shape[0], groups, tile_m).step(counts_all,
                                                                            copy_min_rows)
    out["local_m"] = out["local_m"].tolist()
    return out


class _RawCudaBuffer:
    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {
            "shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2,
        }


class SharedBuffers:
    """Named device buffers on every rank, each mapped by all ranks of the node."""

    def __init__(self, sizes: dict, *, rank: int, world: int, group=None):
        import torch
        import torch.distributed as dist

        self._lib = _capi.load()
        self.rank, self.world = rank, world
        dev = torch.device("cuda", torch.cuda.current_device())
        names = list(sizes)
        self._own, self._opened = [], []
        self.local = {}       # name -> uint8 tensor over the own buffer
        self.bases = {}       # name -> int64 device tensor [world] of base pointers
        handles = torch.zeros(len(names), 64, dtype=torch.uint8)
        own_ptr = {}
        for i, name in enumerate(names):
            nbytes = max(256, int(sizes[name]))
            ptr, buf = C.c_void_p(), (C.c_uint8 * 64)()
            _capi.check(self._lib.bmoe_peer_alloc(nbytes, C.byref(ptr), buf), "bmoe_peer_alloc")
            self._own.append(ptr.value)
            own_ptr[name] = ptr.value
            handles[i] = torch.tensor(list(buf), dtype=torch.uint8)
            self.local[name] = torch.as_tensor(_RawCudaBuffer(ptr.value, nbytes), device=dev)
            self.local[name].zero_()
        table = {name: [0] * world for name in names}
        for name in names:
            table[name][rank] = own_ptr[name]
        if world > 1:
            gathered = torch.zeros(world, len(names), 64, dtype=torch.uint8, device=dev)
            dist.all_gather_into_tensor(gathered.view(-1), handles.to(dev).view(-1), group=group)
            gathered = gathered.cpu()
            for r in range(world):
                if r == rank:
                    continue
                for i, name in enumerate(names):
                    raw = (C.c_uint8 * 64)(*gathered[r, i].tolist())
                    ptr = C.c_void_p()
                    _capi.check(self._lib.bmoe_peer_open(raw, C.byref(ptr)), "bmoe_peer_open")
                    self._opened.append(ptr.value)
                    table[name][r] = ptr.value
        self.host_bases = table     # name -> [world] pointers, for host-issued peer copies
        for name in names:
            self.bases[name] = torch.tensor(table[name], dtype=torch.int64, device=dev)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier(group=group)   # every buffer is zeroed before anyone writes flags

    def close(self):
        import torch

        torch.cuda.synchronize()
        for p in self._opened:
            self._lib.bmoe_peer_close(p)
        self._opened = []
        self.local = {}
        for p in self._own:
            self._lib.bmoe_peer_free(p)
        self._own = []


class FusedExpertParallelLayer:
    def __init__(self, owner: Sequence[int], n: int, k: int, *, rank: int, world: int,
                 rows_cap: int, assignments_cap: int, group=None, scheduler="dynamic_queue",
                 exchange_groups: int = 4, dispatch_ctas: int = 0, wait_budget_ns: int = 0,
                 push_results: bool = True, exchange_sms: int = 16,
                 expert_parts: Sequence[int] | None = None, bulk_copies: bool = False,
                 copy_engine_min_bytes: int = 0, device_plan: bool = True,
                 send_once: bool = False, **plan_options):
        """``rows_cap``: packed rows this rank can own; ``assignments_cap``: local
        assignments (tokens x top_k) per step; ``exchange_groups``: groups the
        experts of a rank are split into for the overlap (1 = no overlap).

        ``expert_parts``: row shards per expert from ``ep.split_and_place_experts``; ``owner``
        then has one entry per SHARD (expert-major), ``local_experts`` lists the expert of
        every local shard (a split expert's weights live on several ranks) and routed rows
        of a split expert are dealt to its shards by assignment index.

        ``exchange_sms`` (even, multi-rank only): SMs the grouped GEMM leaves free for
        the kernel that pushes rows to other GPUs, which then runs as that many
        1024-thread CTAs. An SM whose stores wait for NVLink stalls whatever else runs
        on it, so sharing SMs with GEMM CTAs costs more than giving a few away. The
        GEMM must then be a persistent policy (its grid is what leaves the SMs free).
        0 = share: ``dispatch_ctas`` 256-thread CTAs (default 7/16 of the SMs) that fit
        beside resident GEMM CTAs; any policy.

        ``device_plan``: derive the step's tables from the all-gathered counts with one small
        kernel (``bmoe_ep_plan``) and hand the grouped GEMM its counts in device memory, so
        that a step has no host synchronisation at all (the host only enqueues). Needs
        ``push_results`` and no copy-engine blocks; otherwise the host plans with numpy after
        reading the counts back.

        ``send_once`` (multi-rank only): a token routed to several experts of one other rank
        crosses NVLink once. Of its assignments to that rank the one in the earliest exchange
        group travels as before; for the others the source only writes a small record, and
        the owner's grouped GEMM (a spare warp of every CTA) copies the row that arrived
        onto their packed rows before the group's tiles start. Fewer NVLink bytes (4x at 2
        ranks, 2.1x at 4, 1.4x at 8 for top-8 routing), same result bits.

        ``copy_engine_min_bytes`` (multi-rank only): an (expert, source) block of at least
        this size travels as one peer copy issued by the host (copy engines, no SMs)
        instead of SM stores; 0 (default) = every row goes through the SMs. Measured on
        B200 / NVSwitch the copies lose: the 30-60 copies of a step (5-15 MB each) run one
        after the other at 25-30 us apiece, 160-350 GB/s per GPU, against 360-450 GB/s for
        SM stores from 16 SMs; the path is kept for systems where that differs."""
        import torch

        from .engine import GroupedGemmPlan

        if world > 32:
            raise ValueError("at most 32 ranks")
        self._lib = _capi.load()
        self.owner = [int(o) for o in owner]
        self.experts = len(self.owner)
        self.n, self.k, self.rank, self.world, self.group = n, k, rank, world, group
        self.rows_cap, self.assignments_cap = int(rows_cap), int(assignments_cap)
        self.groups = max(1, min(int(exchange_groups), _capi.EP_MAX_GROUPS)) if world > 1 else 1
        self.local_shards = [e for e in range(self.experts) if self.owner[e] == rank]
        self.expert_parts = None if expert_parts is None else [int(p) for p in expert_parts]
        if self.expert_parts is None:
            self.local_experts = list(self.local_shards)
        else:
            if sum(self.expert_parts) != self.experts or min(self.expert_parts) < 1:
                raise ValueError("owner needs one entry per shard: sum(expert_parts)")
            expert_of_shard = [e for e, p in enumerate(self.expert_parts) for _ in range(p)]
            self.local_experts = [expert_of_shard[s] for s in self.local_shards]
        self.scheduler, self.plan_options = scheduler, dict(plan_options)
        self.dispatch_ctas, self.wait_budget_ns = int(dispatch_ctas), int(wait_budget_ns)
        self.exchange_sms = int(exchange_sms) // 2 * 2 if world > 1 else 0
        if self.exchange_sms:
            if str(scheduler) in ("clc", "auto", "5", "4"):
                raise ValueError("exchange_sms > 0 needs a persistent policy (static or "
                                 "dynamic_queue): one CTA per tile would fill the SMs meant "
                                 "for the exchange kernel")
            sms = torch.cuda.get_device_properties(torch.cuda.current_device()) \
                .multi_processor_count
            pair = self.plan_options.get("cta_group", 0) != 1 and n > 128
            self.plan_options["cta_group"] = 2 if pair else 1
            self.plan_options["cta_count"] = max(1, (sms - self.exchange_sms) // (2 if pair else 1))
        self.push_results = bool(push_results)
        # remote rows as TMA bulk copies through shared-memory stages (needs exchange_sms)
        self.bulk_copies = bool(bulk_copies)
        self.tile_m = 128 if plan_options.get("cta_group") == 1 else 256
        self.plan = GroupedGemmPlan()
        self._planner = StepPlanner(self.owner, rank, world, self.groups, self.tile_m)
        self.launches = 0
        self.epoch = 0
        dev = torch.device("cuda", torch.cuda.current_device())
        self.dev = dev
        flag_slots = 2 * (_capi.EP_MAX_GROUPS + 1) * world   # pushed rows | peer copies
        self.copy_min_rows = 0
        if world > 1 and copy_engine_min_bytes > 0:
            self.copy_min_rows = max(1, -(-int(copy_engine_min_bytes) // (k * 2)))
        # every rank loads its kernels before the first step: the step's bounded waits
        # assume that all ranks launch within the wait budget
        _capi.check(self._lib.bmoe_preload_kernels(), "bmoe_preload_kernels")
        # (a persistent grid only: the warps that copy the rows stay until the last group's
        # flags are up, which one-CTA-per-tile launches cannot afford)
        self.send_once = bool(send_once) and world > 1 and not self.copy_min_rows and \
            str(scheduler) in ("expert_order", "baseline", "static_persistent", "static",
                               "sorted_static", "compacted", "dynamic_queue", "dynamic",
                               "0", "1", "2", "3")
        self._record_cap = max(1, self.assignments_cap)
        sizes = {"a": self.rows_cap * k * 2, "d": self.rows_cap * n * 2, "origin": self.rows_cap * 8,
                 "y": self.assignments_cap * n * 2, "flags": flag_slots * 4}
        if self.send_once:
            # record lists {row that arrived, row to fill} per (group, source), written by the
            # sources, and their lengths
            sizes["dups"] = self.groups * world * self._record_cap * 8
            sizes["dup_count"] = _capi.EP_MAX_GROUPS * world * 4
        self.shared = SharedBuffers(sizes, rank=rank, world=world, group=group)
        loc = self.shared.local
        self.a = loc["a"].view(torch.bfloat16)[:self.rows_cap * k].view(self.rows_cap, k)
        self.d = loc["d"].view(torch.bfloat16)[:self.rows_cap * n].view(self.rows_cap, n)
        self.y = loc["y"].view(torch.bfloat16)[:self.assignments_cap * n] \
            .view(self.assignments_cap, n)
        # per-step tables: int64 row_base[E] | uint8 group_of[E] | uint8 group_local[E] |
        # (4-aligned) uint32 first packed row of every local expert [E]
        # | uint32 bucket offsets [MAX_GROUPS + 3] | uint32 copy mask [MAX_GROUPS]
        # | (8-aligned) int64 staging row base [E]
        self._off_expert_row = (10 * self.experts + 3) // 4 * 4
        self._off_buckets = self._off_expert_row + 4 * self.experts
        self._off_copy_mask = self._off_buckets + 4 * (_capi.EP_MAX_GROUPS + 3)
        self._off_staging = (self._off_copy_mask + 4 * _capi.EP_MAX_GROUPS + 7) // 8 * 8
        # | uint32 rows per local expert [E] | uint32 totals [2] (device planner only)
        self._off_local_rows = self._off_staging + 8 * self.experts
        self._off_totals = self._off_local_rows + 4 * self.experts
        self._table_bytes = self._off_totals + 8
        self._stage = torch.empty(self._table_bytes, dtype=torch.uint8).pin_memory()
        self._tables = torch.empty(self._table_bytes, dtype=torch.uint8, device=dev)
        self._owner_dev = torch.tensor(self.owner, dtype=torch.int32, device=dev)
        # uint32 scratch zeroed every step: cursor[E] | group_done[MAX_GROUPS] | return
        # counter | claim counters of the remote, the local and the staging copy launch
        # [MAX_GROUPS + 2 each] | bucket fill [MAX_GROUPS + 2]
        # | send-once: record fill [world * MAX_GROUPS] | its launch's arrival counter
        # | expansion claim counters [MAX_GROUPS * world] | expansion done [MAX_GROUPS]
        g2 = _capi.EP_MAX_GROUPS + 2
        self._off_dup_fill = self.experts + _capi.EP_MAX_GROUPS + 1 + 4 * g2
        self._off_dup_done = self._off_dup_fill + world * _capi.EP_MAX_GROUPS
        self._off_expand_next = self._off_dup_done + 1
        self._off_expand_done = self._off_expand_next + world * _capi.EP_MAX_GROUPS
        self._scratch = torch.zeros(self._off_expand_done + _capi.EP_MAX_GROUPS,
                                    dtype=torch.int32, device=dev)
        if self.send_once:
            self._row_of = torch.full((self._record_cap,), -1, dtype=torch.int64, device=dev)
            self._primary = torch.full((self._record_cap,), -1, dtype=torch.int32, device=dev)
        self._entries = torch.empty(max(1, self.assignments_cap) * 16, dtype=torch.uint8,
                                    device=dev)
        self._wait_status = torch.zeros(1, dtype=torch.int32, device=dev)
        if self.expert_parts is not None:
            parts = torch.tensor(self.expert_parts, dtype=torch.int64)
            self._parts_dev = parts.to(dev)
            self._shard_base_dev = (torch.cumsum(parts, 0) - parts).to(dev)
        self._comm = torch.cuda.Stream(device=dev)
        self._ev_start = torch.cuda.Event()
        self._ev_comm = torch.cuda.Event()
        self.routes = None
        persistent = str(scheduler) in ("expert_order", "baseline", "static_persistent", "static",
                                        "sorted_static", "compacted", "dynamic_queue", "dynamic",
                                        "0", "1", "2", "3")
        self.device_plan = bool(device_plan) and self.push_results and not self.copy_min_rows \
            and persistent and self.experts <= 4096 and len(self.local_shards) > 0 \
            and not self.plan_options.get("hybrid_tail_tiles")
        if self.device_plan:
            order = np.lexsort((np.arange(self.experts), np.asarray(self.owner)))
            self._order_dev = torch.tensor(order, dtype=torch.int32, device=dev)
            self._counts_all_dev = torch.zeros(world * self.experts, dtype=torch.int64, device=dev)
            self._tables.zero_()
        self._last_local_m = None
        self.copy_bytes = 0      # bytes of the last step that went as peer copies
        self._copy_streams_used = []
        if self.copy_min_rows:
            # staging for the rows of copy-engine blocks (worst case: every local assignment)
            self._staging = torch.empty(max(1, self.assignments_cap), k, dtype=torch.bfloat16,
                                        device=dev)
            self._staging_base = torch.tensor([self._staging.data_ptr()] * world,
                                              dtype=torch.int64, device=dev)
            self._pack = torch.cuda.Stream(device=dev)
            self._ev_pack = torch.cuda.Event()
            # one stream per destination: blocks for one rank stay in order (its flag copy
            # follows its data), blocks for different ranks go out side by side
            self._copy_streams = [torch.cuda.Stream(device=dev) for _ in range(world)]
            self._copy_stream_table = (C.c_void_p * world)(
                *[st.cuda_stream for st in self._copy_streams])
            self._ev_copies = [torch.cuda.Event() for _ in range(world)]
            self._copy_streams_used = []
            # the flag words the 4-byte copies read: word i holds epoch _epoch_base + i
            self._epoch_base = 0
            self._epoch_words = torch.arange(0, 1 << 16, dtype=torch.int32, device=dev)

    def close(self):
        self.plan.close()
        self.shared.close()

    # ------------------------------------------------------------- launches --
    def _scratch_ptr(self, word: int) -> int:
        return self._scratch.data_ptr() + 4 * word

    def _route(self, flat_ids, top_k, stream, routes):
        e, g2 = self.experts, _capi.EP_MAX_GROUPS + 2
        t = self._tables.data_ptr()
        staged = self.copy_min_rows > 0
        args = _capi.EpRouteArgs(
            expert_ids_dev=flat_ids.data_ptr(), row_base_dev=t,
            owner_dev=self._owner_dev.data_ptr(), group_of_dev=t + 8 * e,
            cursor_dev=self._scratch_ptr(0),
            origin_bases_dev=self.shared.bases["origin"].data_ptr(),
            entries_dev=self._entries.data_ptr(), bucket_offset_dev=t + self._off_buckets,
            bucket_fill_dev=self._scratch_ptr(e + _capi.EP_MAX_GROUPS + 1 + 3 * g2),
            staging_row_base_dev=(t + self._off_staging) if staged else None,
            staging_rows_cap=int(self._staging.shape[0]) if staged else 0,
            dst_rank_out_dev=routes[0].data_ptr() if routes else None,
            dst_row_out_dev=(self._row_of.data_ptr() if self.send_once
                             else routes[1].data_ptr() if routes else None),
            primary_out_dev=self._primary.data_ptr() if self.send_once else None,
            assignments=int(flat_ids.numel()), rows_cap=self.rows_cap, top_k=top_k,
            experts=e, ranks=self.world, self=self.rank, groups=self.groups,
            stream=stream.cuda_stream or None)
        _capi.check(self._lib.bmoe_ep_route(C.byref(args)), "bmoe_ep_route")
        if flat_ids.numel():
            self.launches += 1
        if self.send_once:
            # one record per duplicate in the owner's memory, and the list lengths
            dup = _capi.EpDuplicatesArgs(
                expert_ids_dev=flat_ids.data_ptr(), owner_dev=self._owner_dev.data_ptr(),
                group_of_dev=t + 8 * e, primary_dev=self._primary.data_ptr(),
                row_of_dev=self._row_of.data_ptr(),
                record_bases_dev=self.shared.bases["dups"].data_ptr(),
                count_bases_dev=self.shared.bases["dup_count"].data_ptr(),
                fill_dev=self._scratch_ptr(self._off_dup_fill),
                done_counter_dev=self._scratch_ptr(self._off_dup_done),
                assignments=int(flat_ids.numel()), record_cap=self._record_cap, experts=e,
                ranks=self.world, self=self.rank, groups=self.groups,
                stream=stream.cuda_stream or None)
            _capi.check(self._lib.bmoe_ep_duplicates(C.byref(dup)), "bmoe_ep_duplicates")
            self.launches += 1
            if routes:
                routes[1].copy_(self._row_of[:routes[1].numel()])

    def _dispatch(self, x, assignments, mode, stream):
        e, g2 = self.experts, _capi.EP_MAX_GROUPS + 2
        remote = mode == _capi.EP_REMOTE
        pack = mode == _capi.EP_PACK
        claim_set = 0 if remote else (2 if pack else 1)
        args = _capi.EpDispatchArgs(
            x_dev=x.data_ptr(), entries_dev=self._entries.data_ptr(),
            bucket_offset_dev=self._tables.data_ptr() + self._off_buckets,
            a_bases_dev=(self._staging_base if pack else self.shared.bases["a"]).data_ptr(),
            flag_bases_dev=self.shared.bases["flags"].data_ptr(),
            group_done_dev=self._scratch_ptr(e),
            chunk_next_dev=self._scratch_ptr(e + _capi.EP_MAX_GROUPS + 1 + claim_set * g2),
            assignments=assignments, tokens=int(x.shape[0]),
            rows_cap=int(self._staging.shape[0]) if pack else self.rows_cap,
            row_bytes=self.k * 2, ranks=self.world, self=self.rank, groups=self.groups,
            mode=mode, epoch=self.epoch,
            max_ctas=(self.exchange_sms or self.dispatch_ctas) if remote else 0,
            block_threads=1024 if (remote and self.exchange_sms) else 256,
            cluster=2 if (remote and self.exchange_sms) else 0,
            bulk_copies=1 if (remote and self.exchange_sms and self.bulk_copies) else 0,
            status_dev=self._wait_status.data_ptr(),
            stream=stream.cuda_stream or None,
            bucket_fill_dev=(self._scratch_ptr(e + _capi.EP_MAX_GROUPS + 1 + 3 * g2)
                             if self.send_once else None))
        _capi.check(self._lib.bmoe_ep_dispatch(C.byref(args)), "bmoe_ep_dispatch")
        self.launches += 1

    def _send_copies(self, x, step, mine, assignments):
        """Packs the rows of this step's copy-engine blocks into the staging buffer (one
        launch on a stream of its own) and enqueues one peer copy per block plus one
        4-byte flag copy per (destination, group), each destination on its own stream."""
        import torch

        experts = step["copy_experts"]
        self._copy_streams_used = []
        self.copy_bytes = 0
        if experts.size == 0:
            return
        self._pack.wait_event(self._ev_start)
        timed = getattr(self, "_timing_copies", False)
        if timed:
            self._copy_marks = [torch.cuda.Event(enable_timing=True)]
            self._copy_marks[0].record(self._pack)
        self._dispatch(x, assignments, _capi.EP_PACK, self._pack)
        self._ev_pack.record(self._pack)
        if timed:
            self._copy_marks.append(torch.cuda.Event(enable_timing=True))
            self._copy_marks[1].record(self._pack)
        if self.epoch - self._epoch_base >= self._epoch_words.numel():
            torch.cuda.synchronize()
            self._epoch_base = self.epoch
            self._epoch_words.copy_(torch.arange(self.epoch, self.epoch + self._epoch_words.numel(),
                                                 dtype=torch.int64).to(torch.int32))
        row_bytes = self.k * 2
        owners = self._planner.owner_a[experts]
        groups = step["group_of"][experts].astype(np.int64)
        a_base = np.asarray(self.shared.host_bases["a"], dtype=np.uint64)
        flag_base = np.asarray(self.shared.host_bases["flags"], dtype=np.uint64)
        # a flag copy after the last block of every (group, destination) run
        last_of_run = np.ones(experts.size, dtype=bool)
        last_of_run[:-1] = (owners[1:] != owners[:-1]) | (groups[1:] != groups[:-1])
        items = np.zeros(experts.size + int(last_of_run.sum()), dtype=_capi.COPY_ITEM_DTYPE)
        at = np.arange(experts.size) + np.concatenate(([0], np.cumsum(last_of_run)[:-1]))
        items["dst"][at] = a_base[owners] + step["row_base"][experts].astype(np.uint64) * np.uint64(row_bytes)
        items["src"][at] = np.uint64(self._staging.data_ptr()) + \
            step["staging_row_base"][experts].astype(np.uint64) * np.uint64(row_bytes)
        items["bytes"][at] = mine[experts].astype(np.uint64) * np.uint64(row_bytes)
        items["stream"][at] = owners
        flag_at = at[last_of_run] + 1
        plane = _capi.ep_copy_flags(self.world)
        slots = plane + groups[last_of_run] * self.world + self.rank
        items["dst"][flag_at] = flag_base[owners[last_of_run]] + slots.astype(np.uint64) * np.uint64(4)
        items["src"][flag_at] = np.uint64(self._epoch_words.data_ptr()
                                          + 4 * (self.epoch - self._epoch_base))
        items["bytes"][flag_at] = 4
        items["stream"][flag_at] = owners[last_of_run]
        used = sorted(set(int(o) for o in owners))
        for o in used:
            self._copy_streams[o].wait_event(self._ev_pack)
        _capi.check(self._lib.bmoe_peer_copy_batch(items.ctypes.data, len(items),
                                                   self._copy_stream_table, self.world),
                    "bmoe_peer_copy_batch")
        for o in used:
            self._ev_copies[o].record(self._copy_streams[o])
            if timed:
                self._copy_marks.append(torch.cuda.Event(enable_timing=True))
                self._copy_marks[-1].record(self._copy_streams[o])
        self._copy_streams_used = used
        self.copy_bytes = int(items["bytes"][at].sum())

    def _return(self, rows, stream):
        b = self.shared.bases
        args = _capi.EpReturnArgs(
            d_dev=self.d.data_ptr(), origin_dev=self.shared.local["origin"].data_ptr(),
            y_bases_dev=b["y"].data_ptr(), flag_bases_dev=b["flags"].data_ptr(),
            done_counter_dev=self._scratch_ptr(self.experts + _capi.EP_MAX_GROUPS),
            rows=rows, y_rows_cap=self.assignments_cap, row_bytes=self.n * 2, ranks=self.world,
            self=self.rank, flag_slot=_capi.EP_MAX_GROUPS * self.world + self.rank,
            epoch=self.epoch, max_ctas=0, stream=stream.cuda_stream or None)
        _capi.check(self._lib.bmoe_ep_return(C.byref(args)), "bmoe_ep_return")
        self.launches += 1

    # -------------------------------------------------------------- forward --
    def forward(self, x, expert_ids, w_local, record_events=False, topk_weights=None,
                record_routes=False):
        """x [T_local, k]; expert_ids [T_local, top_k] int64; w_local [local experts, n, k].
        Returns y [T_local * top_k, n] in assignment order - a view of the layer's result
        buffer, valid until the next ``forward`` - or, with ``topk_weights``, the weighted
        top-k sum [T_local, n]."""
        import torch
        import torch.distributed as dist

        dev = x.device
        main = torch.cuda.current_stream()
        top_k = int(expert_ids.shape[1])
        flat_ids = expert_ids.reshape(-1).contiguous()
        assignments = int(flat_ids.numel())
        if assignments > self.assignments_cap:
            raise RuntimeError("more assignments than the result buffer holds")
        marks = []

        def mark(name):
            if record_events:
                ev = torch.cuda.Event(enable_timing=True)
                ev.record(main)
                marks.append((name, ev))

        self._timing_copies = bool(record_events)
        self._copy_marks = None
        mark("start")
        # rows per expert (or per row shard of split experts, dealt by assignment index)
        local_counts = torch.empty(self.experts, dtype=torch.int64, device=dev)
        sharded = self.expert_parts is not None
        shard_ids = torch.empty_like(flat_ids) if sharded else None
        _capi.check(
            self._lib.bmoe_ep_count(flat_ids.data_ptr(), assignments,
                                    len(self.expert_parts) if sharded else self.experts,
                                    self._parts_dev.data_ptr() if sharded else None,
                                    self._shard_base_dev.data_ptr() if sharded else None,
                                    self.experts, shard_ids.data_ptr() if sharded else None,
                                    local_counts.data_ptr(), main.cuda_stream or None),
            "bmoe_ep_count")
        self.launches += 1
        self._scratch.zero_()          # cursors and counters of the step; before the host waits
        if sharded:
            flat_ids = shard_ids
        e = self.experts
        step = None
        if self.device_plan:
            # counts stay on the device: all-gather, one planning launch, no read-back
            flat = self._counts_all_dev
            if self.world > 1:
                dist.all_gather_into_tensor(flat, local_counts, group=self.group)
            else:
                flat = local_counts
            t = self._tables.data_ptr()
            args = _capi.EpPlanArgs(
                counts_all_dev=flat.data_ptr(), owner_dev=self._owner_dev.data_ptr(),
                order_dev=self._order_dev.data_ptr(), row_base_dev=t, group_of_dev=t + 8 * e,
                group_local_dev=t + 9 * e, expert_row_dev=t + self._off_expert_row,
                local_rows_dev=t + self._off_local_rows,
                bucket_offset_dev=t + self._off_buckets, totals_dev=t + self._off_totals,
                rows_cap=self.rows_cap, experts=e, ranks=self.world, self=self.rank,
                groups=self.groups, tile_m=self.tile_m, stream=main.cuda_stream or None)
            _capi.check(self._lib.bmoe_ep_plan(C.byref(args)), "bmoe_ep_plan")
            self.launches += 1
            self._last_local_m = None
        else:
            if self.world > 1:
                flat = torch.empty(self.world * self.experts, dtype=torch.int64, device=dev)
                dist.all_gather_into_tensor(flat, local_counts, group=self.group)
                counts_all = flat.reshape(self.world, self.experts).cpu().numpy()
            else:
                counts_all = local_counts.reshape(1, -1).cpu().numpy()
            step = self._planner.step(counts_all, self.copy_min_rows)
            if step["total_local"] > self.rows_cap:
                raise RuntimeError("routed rows exceed the packed buffer capacity")
            stage = self._stage.numpy()
            stage[:8 * e].view(np.int64)[:] = step["row_base"]
            stage[8 * e:9 * e] = step["group_of"]
            stage[9 * e:9 * e + len(step["group_local"])] = step["group_local"]
            local_m = step["local_m"]
            stage[self._off_expert_row:self._off_expert_row + 4 * len(local_m)].view(np.uint32)[:] = \
                np.cumsum(local_m) - local_m
            buckets = step["bucket_offset"]
            stage[self._off_buckets:self._off_buckets + 4 * len(buckets)].view(np.uint32)[:] = buckets
            mask = step["copy_mask"]
            stage[self._off_copy_mask:self._off_copy_mask + 4 * len(mask)].view(np.uint32)[:] = mask
            stage[self._off_staging:self._off_staging + 8 * e].view(np.int64)[:] = \
                step["staging_row_base"]
            self._tables.copy_(self._stage, non_blocking=True)
            self._last_local_m = step["local_m"].tolist()
        self.epoch += 1
        routes = None
        if record_routes:
            routes = (torch.full((assignments,), -1, dtype=torch.int32, device=dev),
                      torch.full((assignments,), -1, dtype=torch.int64, device=dev))
        self.routes = routes
        self._route(flat_ids, top_k, main, routes)
        mark("counts")

        self._ev_start.record(main)       # routes planned: the copy launches may start

        def push_remote():
            # rows bound for other GPUs: side stream, overlapped with everything below
            self._comm.wait_event(self._ev_start)
            if record_events:
                self._remote_marks = (torch.cuda.Event(enable_timing=True),
                                      torch.cuda.Event(enable_timing=True))
                self._remote_marks[0].record(self._comm)
            self._dispatch(x, assignments, _capi.EP_REMOTE, self._comm)
            if record_events:
                self._remote_marks[1].record(self._comm)
            self._ev_comm.record(self._comm)

        # Rows that stay here go in the GEMM's stream. With SMs set aside for the remote
        # pushes the two launches cannot share an SM (registers), so the pushes start
        # first; when they share SMs the local copy goes first, because an SM whose
        # stores wait for NVLink slows this short copy several times.
        if self.world > 1 and self.exchange_sms:
            push_remote()
        # the rows that stay are what the GEMM's stream waits for: their launch goes ahead
        # of the staging launch, which may share the SMs with the start of the GEMM
        self._dispatch(x, assignments, _capi.EP_LOCAL, main)
        if self.copy_min_rows:
            self._send_copies(x, step, counts_all[self.rank], assignments)

        if self.world > 1 and not self.exchange_sms:
            push_remote()
        mark("local_rows")

        total_local = step["total_local"] if step is not None else -1
        if total_local:
            # one A descriptor over the packed buffer, cached B descriptors and (when the
            # epilogue pushes the rows) no D descriptors: a re-plan encodes next to nothing
            if step is None:
                _capi.check(self.plan.initialize_packed_device_counts(
                    self.a, w_local, self._tables.data_ptr() + self._off_local_rows,
                    scheduler=self.scheduler, stream=main, **self.plan_options),
                    "bmoe_plan_initialize")
            else:
                _capi.check(self.plan.initialize_packed(self.a, w_local, self.d, step["local_m"],
                                                        scheduler=self.scheduler, stream=main,
                                                        single_a_map=True,
                                                        results_pushed=self.push_results,
                                                        **self.plan_options),
                            "bmoe_plan_initialize")
            if self.world > 1:
                _capi.check(self.plan.set_gate(self.shared.local["flags"].data_ptr(), self.epoch,
                                               self.world, self.rank,
                                               self._tables.data_ptr() + 9 * e),
                            "bmoe_plan_set_gate")
                if self.copy_min_rows:
                    _capi.check(self.plan.set_gate_copies(self._tables.data_ptr()
                                                          + self._off_copy_mask),
                                "bmoe_plan_set_gate_copies")
                if self.send_once:
                    _capi.check(self.plan.set_expand(
                        self.shared.local["dups"].data_ptr(),
                        self.shared.local["dup_count"].data_ptr(),
                        self._scratch_ptr(self._off_expand_next),
                        self._scratch_ptr(self._off_expand_done), self.a.data_ptr(),
                        self.rows_cap, self.k * 2, self._record_cap, self.groups),
                        "bmoe_plan_set_expand")
            if self.push_results:
                _capi.check(self.plan.set_push(self.shared.local["origin"].data_ptr(),
                                               self._tables.data_ptr() + self._off_expert_row,
                                               self.shared.bases["y"].data_ptr(), self.world,
                                               self.assignments_cap),
                            "bmoe_plan_set_push")
            _capi.check(self.plan.run(main), "bmoe_plan_run")
            self.launches += 3
        mark("gemm")

        if not self.push_results:
            self._return(total_local, main)
        elif self.world > 1:
            self._return(0, main)        # rows already went out of the epilogue: flags only
        if self.world > 1:
            _capi.check(
                self._lib.bmoe_ep_wait_flags(self.shared.local["flags"].data_ptr(),
                                             _capi.EP_MAX_GROUPS * self.world, self.world,
                                             self.rank, self.epoch, self.wait_budget_ns,
                                             self._wait_status.data_ptr(),
                                             main.cuda_stream or None),
                "bmoe_ep_wait_flags")
            self.launches += 1
            main.wait_event(self._ev_comm)
            for o in self._copy_streams_used:   # the staging buffer is free again
                main.wait_event(self._ev_copies[o])
        mark("return")
        y = self.y[:assignments]
        if topk_weights is not None:
            # dropped assignments (expert id out of range) have no result row: skip them
            rows = torch.arange(assignments, device=dev, dtype=torch.int64)
            rows = torch.where((flat_ids >= 0) & (flat_ids < self.experts), rows,
                               torch.full_like(rows, -1)).reshape(-1, top_k)
            out = torch.empty(assignments // top_k, self.n, dtype=x.dtype, device=dev)
            weights = topk_weights.to(torch.float32).contiguous()
            _capi.check(
                self._lib.bmoe_combine_topk(self.shared.bases["y"].data_ptr()
                                            + 8 * self.rank, 1, self.assignments_cap, None,
                                            rows.data_ptr(), weights.data_ptr(),
                                            assignments // top_k, top_k, self.n, out.data_ptr(),
                                            0, main.cuda_stream or None),
                "bmoe_combine_topk")
            self.launches += 1
            y = out
            mark("weighted_sum")
        self._marks = marks
        return y

    @property
    def last_local_m(self):
        """Rows per local expert of the last step (read back on demand when the step was
        planned on the device)."""
        if self._last_local_m is None:
            import torch

            rows = self._tables[self._off_local_rows:self._off_local_rows
                                + 4 * len(self.local_shards)].cpu().numpy().view(np.uint32)
            self._last_local_m = [int(r) for r in rows]
        return self._last_local_m

    def poll(self):
        status, report = self.plan.poll()
        if status not in (_capi.OK, _capi.INVALID_ARGUMENT):
            raise _capi.EngineError(
                status, f"grouped GEMM (site {report.code}, cta {report.cta}, "
                        f"group {report.stage}, rank {report.aux})")
        if self.device_plan:
            totals = self._tables[self._off_totals:self._off_totals + 8].cpu().numpy().view(np.uint32)
            if int(totals[1]) != 0:
                raise RuntimeError(f"routed rows ({int(totals[0])}) exceed the packed buffer "
                                   f"capacity ({self.rows_cap})")
        word = int(self._wait_status.item()) & 0xffffffff
        if word:
            self._wait_status.zero_()   # reported once; the layer stays usable
        if word & 0x40000000:
            raise _capi.EngineError(_capi.DEVICE_TIMEOUT,
                                    f"a bulk copy of exchange group {word & 0xff} did not complete")
        if word:
            raise _capi.EngineError(
                _capi.DEVICE_TIMEOUT,
                f"results of rank {word & 0xff} did not arrive (flag slot {(word >> 8) & 0xffff})")

    def phase_times_ms(self):
        import torch

        torch.cuda.synchronize()
        out = {name: a.elapsed_time(b)
               for (_, a), (name, b) in zip(self._marks[:-1], self._marks[1:])}
        if self.world > 1 and getattr(self, "_remote_marks", None):
            # side stream: runs beside local_rows / gemm, not part of their sum
            out["remote_rows_overlapped"] = self._remote_marks[0].elapsed_time(self._remote_marks[1])
        if getattr(self, "_copy_marks", None):
            # staging launch, then the peer copies on their streams (start of staging to
            # the end of the last copy), beside everything else
            m = self._copy_marks
            out["staging_overlapped"] = m[0].elapsed_time(m[1])
            out["peer_copies_overlapped"] = max(m[0].elapsed_time(end) for end in m[2:])
        return out
