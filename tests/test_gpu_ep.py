"""Expert-parallel layer on GPUs: the row-gather kernel, the single-rank layer
against the plain engine, and (with two or more GPUs) NCCL ranks against the
single-GPU engine, bit for bit."""

import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def test_gather_rows_matches_index_select(engine):
    import torch

    from bmoe_b200 import ep

    ops = ep.CudaOps()
    gen = torch.Generator().manual_seed(3)
    for rows, width in [(1, 8), (1000, 7168), (4097, 2048), (33, 24)]:
        src = torch.randn(rows, width, generator=gen).to(torch.bfloat16).cuda()
        index = torch.randint(0, rows, (rows * 2 + 3,), generator=gen).cuda()
        got = ops.gather_rows(src, index)
        assert torch.equal(got.view(torch.int16), src.index_select(0, index).view(torch.int16))
    # out-of-range entries leave the destination row untouched
    src = torch.ones(4, 8, dtype=torch.bfloat16, device="cuda")
    out = torch.zeros(3, 8, dtype=torch.bfloat16, device="cuda")
    ops.gather_rows(src, torch.tensor([1, 99, -1], device="cuda"), out=out)
    assert out[0].eq(1).all() and out[1:].eq(0).all()


def oracle_combine(y, gates, top_k):
    """CPU oracle of the weighted top-k sum over rows in assignment order."""
    import support
    import torch

    bits = y.cpu().contiguous().view(torch.int16).numpy().view(np.uint16)
    rows = np.arange(bits.shape[0], dtype=np.int64).reshape(-1, top_k)
    out = support.Oracle().combine_topk(bits, rows, gates.cpu().numpy())
    return torch.from_numpy(out.view(np.int16).copy()).view(torch.bfloat16)


def test_combine_topk_is_bit_exact_against_the_oracle(engine):
    import support
    import torch

    from bmoe_b200 import ep

    ops = ep.CudaOps()
    oracle = support.Oracle()
    gen = torch.Generator().manual_seed(11)
    for src_rows, n, tokens, top_k in [(5, 8, 1, 1), (300, 24, 77, 2), (4096, 2048, 700, 8),
                                       (2000, 7168, 130, 4), (900, 264, 55, 9)]:
        src = torch.randn(src_rows, n, generator=gen).to(torch.bfloat16)
        rows = torch.randint(0, src_rows, (tokens, top_k), generator=gen)
        rows[tokens // 2, 0] = -1                      # a dropped assignment
        if tokens > 3:
            rows[3, :] = -1                            # a token with nothing routed
            rows[1, top_k - 1] = src_rows + 5          # out of range: skipped as well
        gates = torch.rand(tokens, top_k, generator=gen)
        src_bits = src.view(torch.int16).numpy().view(np.uint16)
        for weights in (gates, None):
            got = ops.combine_topk(src.cuda(), rows.cuda(),
                                   None if weights is None else weights.cuda())
            want = oracle.combine_topk(src_bits, rows.numpy(),
                                       None if weights is None else weights.numpy())
            got_bits = got.cpu().view(torch.int16).numpy().view(np.uint16)
            assert np.array_equal(got_bits, want), (src_rows, n, tokens, top_k)
    lib = engine._capi.load()
    assert lib.bmoe_combine_topk(None, 1, 1, None, None, None, 4, 2, 8, None, 0, None) != 0
    assert lib.bmoe_combine_topk(None, 1, 1, None, None, None, 0, 2, 8, None, 0, None) == 0


def reference_output(engine, x_all, ids_all, w_all, top_k):
    """Single-GPU engine over all assignments, returned in assignment order."""
    import torch

    experts = w_all.shape[0]
    flat = ids_all.reshape(-1)
    counts = torch.bincount(flat, minlength=experts).tolist()
    order = torch.sort(flat, stable=True).indices
    a = x_all[order // top_k].contiguous().cuda()
    d = torch.zeros(a.shape[0], w_all.shape[1], dtype=torch.bfloat16, device="cuda")
    engine.grouped_gemm(a, w_all.cuda(), d, counts, scheduler="expert_order")
    y = torch.empty_like(d)
    y[order.cuda()] = d
    return y


def make_problem(experts=40, top_k=4, tokens=600, n=512, k=320):
    import torch

    gen = torch.Generator().manual_seed(2026)
    probs = 1.0 / torch.arange(1, experts + 1, dtype=torch.float64)
    probs[7] = 0.0
    ids = torch.multinomial(probs.expand(tokens, -1), top_k, replacement=False, generator=gen)
    x = torch.randn(tokens, k, generator=gen).to(torch.bfloat16)
    w = (torch.randn(experts, n, k, generator=gen) * k ** -0.5).to(torch.bfloat16)
    return ids, x, w


def test_single_rank_layer_equals_plain_engine(engine):
    import torch

    from bmoe_b200 import ep

    ids, x, w = make_problem()
    owner, _ = ep.place_experts(torch.bincount(ids.reshape(-1), minlength=40).tolist(), 1, 512)
    layer = ep.ExpertParallelLayer(owner, 512, 320, rank=0, world=1,
                                   ops=ep.CudaOps(scheduler="dynamic_queue"))
    y = layer.forward(x.cuda(), ids.cuda(), w.cuda())
    layer.ops.poll()
    want = reference_output(engine, x, ids, w, 4)
    assert torch.equal(y.view(torch.int16), want.view(torch.int16))
    gates = torch.rand(ids.shape, generator=torch.Generator().manual_seed(1))
    z = layer.forward(x.cuda(), ids.cuda(), w.cuda(), topk_weights=gates.cuda())
    assert z.shape == (x.shape[0], 512)
    assert torch.equal(z.cpu().view(torch.int16), oracle_combine(want, gates, 4).view(torch.int16))


def test_route_rows_and_single_rank_peer_layer(engine):
    """bmoe_route_rows against index_select / index_copy, and the peer-memory layer
    on one rank (its own buffers only) against the plain engine."""
    import ctypes as C

    import torch

    from bmoe_b200 import ep, ep_peer

    lib = engine._capi.load()
    gen = torch.Generator().manual_seed(5)
    src = torch.randn(300, 512, generator=gen).to(torch.bfloat16).cuda()
    dst = torch.zeros(400, 512, dtype=torch.bfloat16, device="cuda")
    src_row = torch.randint(0, 300, (350,), generator=gen).cuda()
    dst_row = torch.randperm(400, generator=gen)[:350].cuda()
    dst_row[7] = 4000  # out of range: skipped
    bases_s = torch.tensor([src.data_ptr()], dtype=torch.int64, device="cuda")
    bases_d = torch.tensor([dst.data_ptr()], dtype=torch.int64, device="cuda")
    rc = lib.bmoe_route_rows(bases_s.data_ptr(), 1, 300, None, src_row.data_ptr(),
                             bases_d.data_ptr(), 1, 400, None, dst_row.data_ptr(), 350, 1024, 0,
                             None)
    assert rc == 0
    want = torch.zeros_like(dst)
    keep = torch.ones(350, dtype=torch.bool)
    keep[7] = False
    want[dst_row[keep.cuda()]] = src[src_row[keep.cuda()]]
    assert torch.equal(dst.view(torch.int16), want.view(torch.int16))

    ids, x, w = make_problem()
    owner = [0] * 40
    layer = ep_peer.PeerExpertParallelLayer(owner, 512, 320, rank=0, world=1, rows_cap=2400)
    try:
        for _ in range(2):
            y = layer.forward(x.cuda(), ids.cuda(), w.cuda())
        layer.poll()
        want = reference_output(engine, x, ids, w, 4)
        assert torch.equal(y.view(torch.int16), want.view(torch.int16))
        gates = torch.rand(ids.shape, generator=torch.Generator().manual_seed(1))
        z = layer.forward(x.cuda(), ids.cuda(), w.cuda(), topk_weights=gates.cuda())
        assert torch.equal(z.cpu().view(torch.int16),
                           oracle_combine(want, gates, 4).view(torch.int16))
    finally:
        layer.close()


def test_single_rank_fused_layer_and_gate(engine):
    """The overlapped-exchange layer on one rank against the plain engine, the gate of
    the grouped GEMM with flags that are already up, and the bounded waits: a flag
    that nothing raises makes the wait kernel and the gated GEMM give up with a
    status instead of hanging."""
    import torch

    from bmoe_b200 import ep_fused

    ids, x, w = make_problem()
    want = reference_output(engine, x, ids, w, 4)
    for push, opts in ((False, {}), (True, {"cta_group": 1}), (True, {"scheduler": "clc"}),
                       (True, {"device_plan": False})):
        plain = ep_fused.FusedExpertParallelLayer([0] * 40, 512, 320, rank=0, world=1,
                                                  rows_cap=2400, assignments_cap=2400,
                                                  push_results=push, **opts)
        try:
            y = plain.forward(x.cuda(), ids.cuda(), w.cuda())
            plain.poll()
            assert torch.equal(y.view(torch.int16), want.view(torch.int16)), (push, opts)
        finally:
            plain.close()
    # row shards: experts 0 and 3 are dealt to 3 and 2 shards (all on this one rank)
    parts = [3, 1, 1, 2] + [1] * 36
    expert_of_shard = [e for e, p in enumerate(parts) for _ in range(p)]
    sharded = ep_fused.FusedExpertParallelLayer([0] * sum(parts), 512, 320, rank=0, world=1,
                                                rows_cap=2400, assignments_cap=2400,
                                                expert_parts=parts)
    try:
        assert sharded.local_experts == expert_of_shard
        y = sharded.forward(x.cuda(), ids.cuda(), w[sharded.local_experts].cuda())
        sharded.poll()
        assert torch.equal(y.view(torch.int16), want.view(torch.int16))
        per_shard = sharded.last_local_m
        first = int((ids == 0).sum())
        # dealt by assignment index: all rows accounted for, shards about equal
        assert sum(per_shard[:3]) == first
        assert max(per_shard[:3]) <= 1.4 * first / 3 and min(per_shard[:3]) >= 0.6 * first / 3
    finally:
        sharded.close()
    layer = ep_fused.FusedExpertParallelLayer([0] * 40, 512, 320, rank=0, world=1,
                                              rows_cap=2400, assignments_cap=2400)
    try:
        for _ in range(2):
            y = layer.forward(x.cuda(), ids.cuda(), w.cuda(), record_routes=True)
        layer.poll()
        assert torch.equal(y.view(torch.int16), want.view(torch.int16))
        dst_rank, dst_row = layer.routes
        assert dst_rank.eq(0).all() and torch.equal(
            torch.sort(dst_row).values.cpu(), torch.arange(2400))
        gates = torch.rand(ids.shape, generator=torch.Generator().manual_seed(1))
        z = layer.forward(x.cuda(), ids.cuda(), w.cuda(), topk_weights=gates.cuda())
        assert torch.equal(z.cpu().view(torch.int16),
                           oracle_combine(want, gates, 4).view(torch.int16))
        # dropped assignments (expert id -1 or out of range) take part in nothing
        dropped = ids.clone()
        dropped[5, 1] = -1
        dropped[17, :] = 40
        z = layer.forward(x.cuda(), dropped.cuda(), w.cuda(), topk_weights=gates.cuda())
        layer.poll()
        import support
        rows = np.arange(2400, dtype=np.int64).reshape(-1, 4)
        rows[5, 1] = -1
        rows[17, :] = -1
        want_bits = support.Oracle().combine_topk(
            want.cpu().contiguous().view(torch.int16).numpy().view(np.uint16), rows, gates.numpy())
        assert np.array_equal(z.cpu().view(torch.int16).numpy().view(np.uint16), want_bits)
        assert sum(layer.last_local_m) == 2400 - 5
    finally:
        layer.close()

    lib = engine._capi.load()
    assert lib.bmoe_preload_kernels() == 0
    # count kernel: histogram of valid ids, and the shard dealing of split experts
    gen = torch.Generator().manual_seed(8)
    raw = torch.randint(-2, 9, (5000,), generator=gen)               # ids -2..8, experts = 7
    counts = torch.empty(7, dtype=torch.int64, device="cuda")
    assert lib.bmoe_ep_count(raw.cuda().data_ptr(), 5000, 7, None, None, 7, None,
                             counts.data_ptr(), None) == 0
    ok = (raw >= 0) & (raw < 7)
    assert torch.equal(counts.cpu(), torch.bincount(raw[ok], minlength=7))
    parts_t = torch.tensor([1, 3, 1, 2, 1, 1, 1])
    base_t = torch.cumsum(parts_t, 0) - parts_t
    out_ids = torch.empty(5000, dtype=torch.int64, device="cuda")
    counts10 = torch.empty(10, dtype=torch.int64, device="cuda")
    assert lib.bmoe_ep_count(raw.cuda().data_ptr(), 5000, 7, parts_t.cuda().data_ptr(),
                             base_t.cuda().data_ptr(), 10, out_ids.data_ptr(),
                             counts10.data_ptr(), None) == 0
    safe = raw.clamp(0, 6)
    want_ids = torch.where(ok, base_t[safe] + torch.arange(5000) % parts_t[safe],
                           torch.full_like(raw, -1))
    assert torch.equal(out_ids.cpu(), want_ids)
    assert torch.equal(counts10.cpu(), torch.bincount(want_ids[ok], minlength=10))
    assert lib.bmoe_ep_count(raw.cuda().data_ptr(), 5000, 7, None, None, 9, None,
                             counts.data_ptr(), None) != 0            # bins must equal experts

    # wait kernel: rank 1 of 2 never reports -> status word, no hang
    flags = torch.zeros(64, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    assert lib.bmoe_ep_wait_flags(flags.data_ptr(), 32, 2, 0, 1, 2_000_000, status.data_ptr(),
                                  None) == 0
    torch.cuda.synchronize()
    assert (int(status.item()) & 0xffffffff) == (0x80000000 | (32 << 8) | 1)
    flags[33] = 1
    status.zero_()
    assert lib.bmoe_ep_wait_flags(flags.data_ptr(), 32, 2, 0, 1, 2_000_000, status.data_ptr(),
                                  None) == 0
    torch.cuda.synchronize()
    assert int(status.item()) == 0

    # gated GEMM: two groups, "rank 1" delivered group 0 only
    counts = [150, 0, 300, 90]
    gen = torch.Generator().manual_seed(4)
    a = torch.randn(sum(counts), 192, generator=gen).to(torch.bfloat16).cuda()
    wt = (torch.randn(4, 256, 192, generator=gen) * 192 ** -0.5).to(torch.bfloat16).cuda()
    d_plain = torch.zeros(sum(counts), 256, dtype=torch.bfloat16, device="cuda")
    engine.grouped_gemm(a, wt, d_plain, counts, scheduler="dynamic_queue")
    group_of = torch.tensor([0, 0, 1, 1], dtype=torch.uint8, device="cuda")
    flags = torch.zeros(64, dtype=torch.int32, device="cuda")
    flags[0 * 2 + 1] = 5                                   # group 0 from rank 1, epoch 5
    for cta_group in (1, 2):
        d = torch.zeros_like(d_plain)
        plan = engine.GroupedGemmPlan()
        assert plan.initialize_packed(a, wt, d, counts, scheduler="dynamic_queue",
                                      cta_group=cta_group) == 0
        assert plan.set_gate(flags.data_ptr(), 5, 2, 0, group_of.data_ptr()) == 0
        flags[1 * 2 + 1] = 0
        assert plan.run() == 0
        torch.cuda.synchronize()
        status_code, report = plan.poll()
        assert status_code == engine._capi.DEVICE_TIMEOUT and report.code == 11
        assert report.stage == 1 and report.aux == 1       # group 1, rank 1
        flags[1 * 2 + 1] = 5                               # now everything has "arrived"
        assert plan.initialize_packed(a, wt, d, counts, scheduler="dynamic_queue",
                                      cta_group=cta_group) == 0
        assert plan.set_gate(flags.data_ptr(), 5, 2, 0, group_of.data_ptr()) == 0
        assert plan.run() == 0
        torch.cuda.synchronize()
        assert plan.poll()[0] == 0
        assert torch.equal(d.view(torch.int16), d_plain.view(torch.int16))
        plan.close()


def test_route_planning_leaves_no_stale_entry_when_a_row_does_not_fit(engine):
    """A packed buffer that is too short for the routed rows (an inconsistent table): the
    assignments that do not fit reserve their bucket slot all the same, and that slot must
    then hold an entry no rank owns, not whatever an earlier step left there - the copy
    kernels skip such entries, so nothing is written outside the buffer."""
    import ctypes as C

    import torch

    from bmoe_b200 import ep_fused

    cap = engine._capi
    lib = cap.load()
    experts, top_k, tokens, groups = 6, 2, 40, 2
    gen = torch.Generator().manual_seed(3)
    ids = torch.multinomial(torch.ones(experts).expand(tokens, -1), top_k, generator=gen)
    flat = ids.reshape(-1).contiguous().cuda()
    counts = torch.bincount(flat.cpu(), minlength=experts).numpy().reshape(1, -1)
    step = ep_fused.plan_step(counts, [0] * experts, 0, groups)
    assignments = tokens * top_k
    rows_cap = assignments - 25                       # 25 rows do not fit
    row_base = torch.from_numpy(step["row_base"]).cuda()
    owner = torch.zeros(experts, dtype=torch.int32, device="cuda")
    group_of = torch.from_numpy(step["group_of"]).cuda()
    cursor = torch.zeros(experts, dtype=torch.int32, device="cuda")
    origin = torch.full((assignments,), -1, dtype=torch.int64, device="cuda")
    origin_bases = torch.tensor([origin.data_ptr()], dtype=torch.int64, device="cuda")
    stale = np.zeros(assignments, dtype=[("token", "<u4"), ("to", "<u4"), ("row", "<u4"), ("pad", "<u4")])
    stale["row"] = 7                                   # a valid-looking entry from "last step"
    entries = torch.from_numpy(stale.view(np.uint8).copy()).cuda()
    buckets = torch.from_numpy(step["bucket_offset"].astype(np.int32)).cuda()
    fill = torch.zeros(groups + 2, dtype=torch.int32, device="cuda")
    args = cap.EpRouteArgs(
        expert_ids_dev=flat.data_ptr(), row_base_dev=row_base.data_ptr(), owner_dev=owner.data_ptr(),
        group_of_dev=group_of.data_ptr(), cursor_dev=cursor.data_ptr(),
        origin_bases_dev=origin_bases.data_ptr(), entries_dev=entries.data_ptr(),
        bucket_offset_dev=buckets.data_ptr(), bucket_fill_dev=fill.data_ptr(),
        dst_rank_out_dev=None, dst_row_out_dev=None, assignments=assignments, rows_cap=rows_cap,
        top_k=top_k, experts=experts, ranks=1, self=0, groups=groups, stream=None,
        staging_row_base_dev=None, staging_rows_cap=0)
    assert lib.bmoe_ep_route(C.byref(args)) == 0
    torch.cuda.synchronize()
    got = entries.cpu().numpy().view(stale.dtype)
    fits = got["to"] == 0
    assert int(fits.sum()) == rows_cap and np.all(got["row"][fits] < rows_cap)
    assert sorted(got["row"][fits].tolist()) == list(range(rows_cap))
    assert np.all(got["to"][~fits] == 0xFFFFFFFF) and int((~fits).sum()) == 25
    # the copy kernel walks all entries and touches nothing beyond the short buffer
    k = 64
    x = torch.randn(tokens, k, generator=gen).to(torch.bfloat16).cuda()
    a = torch.zeros(assignments, k, dtype=torch.bfloat16, device="cuda")
    a_bases = torch.tensor([a.data_ptr()], dtype=torch.int64, device="cuda")
    claims = torch.zeros(groups + 2, dtype=torch.int32, device="cuda")
    dargs = cap.EpDispatchArgs(
        x_dev=x.data_ptr(), entries_dev=entries.data_ptr(), bucket_offset_dev=buckets.data_ptr(),
        a_bases_dev=a_bases.data_ptr(), flag_bases_dev=None, group_done_dev=None,
        chunk_next_dev=claims.data_ptr(), assignments=assignments, tokens=tokens,
        rows_cap=rows_cap, row_bytes=k * 2, ranks=1, self=0, groups=groups, mode=cap.EP_LOCAL,
        epoch=1, max_ctas=0, block_threads=0, cluster=0, bulk_copies=0, status_dev=None,
        stream=None)
    assert lib.bmoe_ep_dispatch(C.byref(dargs)) == 0
    torch.cuda.synchronize()
    assert a[rows_cap:].eq(0).all()
    want = x[torch.from_numpy(got["token"][fits].astype(np.int64)).cuda()]
    assert torch.equal(a[torch.from_numpy(got["row"][fits].astype(np.int64)).cuda()].view(torch.int16),
                       want.view(torch.int16))


def test_gemm_copies_duplicate_rows_before_their_group_starts(engine):
    """Send-once exchange, owner's side, on one GPU with the flags already up: the record
    lists name rows that did not travel (here: left as NaN) and the rows to copy them from;
    warp 3 of the launch's CTAs fills them and the gate holds every group back until its
    list has been carried out. Output and the packed buffer must equal the run on the fully
    populated buffer."""
    import torch

    counts = [300, 40, 0, 260, 129]
    n, k, ranks, groups, cap = 256, 192, 2, 2, 64
    gen = torch.Generator().manual_seed(12)
    a_full = torch.randn(sum(counts), k, generator=gen).to(torch.bfloat16)
    wt = (torch.randn(len(counts), n, k, generator=gen) * k ** -0.5).to(torch.bfloat16).cuda()
    group_of = torch.tensor([0, 0, 0, 1, 1], dtype=torch.uint8, device="cuda")
    first_row = np.cumsum([0] + counts[:-1])
    # duplicates: rows of group-1 experts copied from group-0 rows, and inside a group; a
    # source row is always one that travelled (never itself a duplicate)
    pairs = {0: [(5, 310), (7, 9), (299, 320)], 1: [(5, 345), (7, 600), (400, 401), (8, 728)]}
    for g in (0, 1):
        for src, dst in pairs[g]:
            a_full[dst] = a_full[src]
    gapped = a_full.clone()
    for g in (0, 1):
        for _, dst in pairs[g]:
            gapped[dst] = float("nan")
    d_want = torch.zeros(sum(counts), n, dtype=torch.bfloat16, device="cuda")
    engine.grouped_gemm(a_full.cuda(), wt, d_want, counts, scheduler="dynamic_queue")
    records = np.zeros((groups, ranks, cap, 2), dtype=np.uint32)
    lengths = np.zeros((groups, ranks), dtype=np.uint32)
    for g in (0, 1):
        records[g, 1, :len(pairs[g])] = pairs[g]
        lengths[g, 1] = len(pairs[g])
    records_dev = torch.from_numpy(records.view(np.int32)).cuda()
    lengths_dev = torch.from_numpy(lengths.view(np.int32)).cuda()
    flags = torch.zeros(64, dtype=torch.int32, device="cuda")
    flags[0 * ranks + 1] = 9
    flags[1 * ranks + 1] = 9
    for cta_group, policy in ((1, "dynamic_queue"), (2, "expert_order"), (2, "dynamic_queue")):
        a_dev = gapped.clone().cuda()
        d = torch.zeros_like(d_want)
        claims = torch.zeros(groups * ranks, dtype=torch.int32, device="cuda")
        done = torch.zeros(groups, dtype=torch.int32, device="cuda")
        plan = engine.GroupedGemmPlan()
        try:
            assert plan.initialize_packed(a_dev, wt, d, counts, scheduler=policy,
                                          cta_group=cta_group) == 0
            assert plan.set_gate(flags.data_ptr(), 9, ranks, 0, group_of.data_ptr()) == 0
            assert plan.set_expand(records_dev.data_ptr(), lengths_dev.data_ptr(),
                                   claims.data_ptr(), done.data_ptr(), a_dev.data_ptr(),
                                   a_dev.shape[0], k * 2, cap, groups) == 0
            assert plan.run() == 0
            status, report = plan.poll()
            assert status == 0, (report.code, report.stage, report.aux)
        finally:
            plan.close()
        assert done.cpu().tolist() == [len(pairs[0]), len(pairs[1])]
        assert torch.equal(a_dev.cpu().view(torch.int16), a_full.view(torch.int16))
        assert torch.equal(d.view(torch.int16), d_want.view(torch.int16)), (cta_group, policy)
    # a list that claims more records than were ever written for it: bounded wait, status
    lengths_dev[1, 1] = 50
    records_dev[1, 1, 4:50] = 0x7fffffff            # rows out of range: skipped, still counted
    a_dev = gapped.clone().cuda()
    d = torch.zeros_like(d_want)
    claims = torch.zeros(groups * ranks, dtype=torch.int32, device="cuda")
    done = torch.zeros(groups, dtype=torch.int32, device="cuda")
    plan = engine.GroupedGemmPlan()
    try:
        assert plan.initialize_packed(a_dev, wt, d, counts, scheduler="dynamic_queue") == 0
        assert plan.set_gate(flags.data_ptr(), 9, ranks, 0, group_of.data_ptr()) == 0
        assert plan.set_expand(records_dev.data_ptr(), lengths_dev.data_ptr(), claims.data_ptr(),
                               done.data_ptr(), a_dev.data_ptr(), a_dev.shape[0], k * 2, cap,
                               groups) == 0
        assert plan.run() == 0 and plan.poll()[0] == 0
        assert done.cpu().tolist() == [len(pairs[0]), 50]
        assert torch.equal(d.view(torch.int16), d_want.view(torch.int16))
        assert plan.set_expand(None, None, None, None, None, 0, 0, 0, 0) == 0
    finally:
        plan.close()


def test_device_planner_equals_host_planner(engine):
    """bmoe_ep_plan (the step tables derived on the device, so that a step needs no host
    synchronisation) against the numpy planner, table for table, over random count
    matrices, owner maps, group counts and tile heights - including owners without
    experts, empty experts and a single rank."""
    import ctypes as C

    import torch

    from bmoe_b200 import ep_fused

    cap = engine._capi
    lib = cap.load()
    rng = np.random.default_rng(77)
    for trial in range(40):
        world = int(rng.integers(1, 9))
        experts = int(rng.integers(1, 300)) if trial % 5 else int(rng.integers(1000, 4097))
        groups = int(rng.integers(1, cap.EP_MAX_GROUPS + 1))
        tile_m = int(rng.choice([128, 256, 16]))
        owner = rng.integers(0, world, size=experts)
        if world > 2:
            owner[owner == 1] = 0                      # a rank that owns nothing
        counts_all = (rng.integers(0, 900, size=(world, experts)) *
                      (rng.random((world, experts)) > 0.3)).astype(np.int64)
        order = np.lexsort((np.arange(experts), owner))
        dev = "cuda"
        counts_dev = torch.from_numpy(counts_all).to(dev)
        owner_dev = torch.from_numpy(owner.astype(np.int32)).to(dev)
        order_dev = torch.from_numpy(order.astype(np.int32)).to(dev)
        for rank in sorted(set([0, world - 1, int(rng.integers(0, world))])):
            want = ep_fused.plan_step(counts_all, owner.tolist(), rank, groups, tile_m)
            n_local = len(want["local_experts"])
            row_base = torch.full((experts,), -7, dtype=torch.int64, device=dev)
            group_of = torch.full((experts,), 255, dtype=torch.uint8, device=dev)
            group_local = torch.full((max(1, experts),), 255, dtype=torch.uint8, device=dev)
            expert_row = torch.zeros(max(1, experts), dtype=torch.int32, device=dev)
            local_rows = torch.zeros(max(1, experts), dtype=torch.int32, device=dev)
            buckets = torch.zeros(cap.EP_MAX_GROUPS + 3, dtype=torch.int32, device=dev)
            totals = torch.zeros(2, dtype=torch.int32, device=dev)
            rows_cap = int(sum(want["local_m"])) + (0 if trial % 7 else -1)
            args = cap.EpPlanArgs(
                counts_all_dev=counts_dev.data_ptr(), owner_dev=owner_dev.data_ptr(),
                order_dev=order_dev.data_ptr(), row_base_dev=row_base.data_ptr(),
                group_of_dev=group_of.data_ptr(), group_local_dev=group_local.data_ptr(),
                expert_row_dev=expert_row.data_ptr(), local_rows_dev=local_rows.data_ptr(),
                bucket_offset_dev=buckets.data_ptr(), totals_dev=totals.data_ptr(),
                rows_cap=max(0, rows_cap), experts=experts, ranks=world, self=rank,
                groups=groups, tile_m=tile_m, stream=None)
            assert lib.bmoe_ep_plan(C.byref(args)) == 0
            torch.cuda.synchronize()
            key = (trial, world, experts, groups, tile_m, rank)
            assert np.array_equal(row_base.cpu().numpy(), want["row_base"]), key
            assert np.array_equal(group_of.cpu().numpy(), want["group_of"]), key
            assert np.array_equal(group_local.cpu().numpy()[:n_local], want["group_local"]), key
            local_m = np.asarray(want["local_m"], dtype=np.int64)
            assert np.array_equal(local_rows.cpu().numpy()[:n_local], local_m), key
            assert np.array_equal(expert_row.cpu().numpy()[:n_local],
                                  np.cumsum(local_m) - local_m), key
            assert np.array_equal(buckets.cpu().numpy()[:groups + 3],
                                  want["bucket_offset"].astype(np.int64)), key
            got_totals = totals.cpu().numpy()
            assert int(got_totals[0]) == int(local_m.sum()), key
            assert int(got_totals[1]) == (1 if local_m.sum() > max(0, rows_cap) else 0), key
    bad = cap.EpPlanArgs(experts=5000, ranks=1, groups=1, tile_m=128)
    assert lib.bmoe_ep_plan(C.byref(bad)) == cap.INVALID_ARGUMENT


def _ep_worker(rank, world, port, tmpdir):
    for p in (ROOT, ROOT / "tests", ROOT / "oracle"):
        sys.path.insert(0, str(p))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch
    import torch.distributed as dist

    import bmoe_b200 as engine
    from bmoe_b200 import ep

    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world,
                            device_id=torch.device("cuda", rank))
    try:
        ids, x, w = make_problem()
        tokens = x.shape[0]
        owner, _ = ep.place_experts(torch.bincount(ids.reshape(-1), minlength=40).tolist(),
                                    world, 512)
        lo, hi = tokens * rank // world, tokens * (rank + 1) // world
        want = reference_output(engine, x, ids, w, 4)[lo * 4:hi * 4]
        gates = torch.rand(ids.shape, generator=torch.Generator().manual_seed(1))[lo:hi]
        want_z = oracle_combine(want, gates, 4)
        same = True
        for groups, opts in ((1, {}), (3, {"cta_group": 2, "cta_count": 60})):
            layer = ep.ExpertParallelLayer(owner, 512, 320, rank=rank, world=world,
                                           ops=ep.CudaOps(scheduler="dynamic_queue", **opts),
                                           pipeline_groups=groups)
            for _ in range(2):
                y = layer.forward(x[lo:hi].cuda(), ids[lo:hi].cuda(),
                                  w[layer.local_experts].cuda())
            layer.ops.poll()
            same = same and torch.equal(y.view(torch.int16), want.view(torch.int16))
            if groups == 1:
                z = layer.forward(x[lo:hi].cuda(), ids[lo:hi].cuda(),
                                  w[layer.local_experts].cuda(), topk_weights=gates.cuda())
                same = same and torch.equal(z.cpu().view(torch.int16), want_z.view(torch.int16))
        from bmoe_b200 import ep_peer

        peer = ep_peer.PeerExpertParallelLayer(owner, 512, 320, rank=rank, world=world,
                                               rows_cap=2400, scheduler="clc")
        for _ in range(3):
            y = peer.forward(x[lo:hi].cuda(), ids[lo:hi].cuda(), w[peer.local_experts].cuda())
        peer.poll()
        same = same and torch.equal(y.view(torch.int16), want.view(torch.int16))
        for _ in range(2):
            z = peer.forward(x[lo:hi].cuda(), ids[lo:hi].cuda(), w[peer.local_experts].cuda(),
                             topk_weights=gates.cuda())
        same = same and torch.equal(z.cpu().view(torch.int16), want_z.view(torch.int16))
        from bmoe_b200 import ep_fused

        parts, shard_owner, _ = ep.split_and_place_experts(
            torch.bincount(ids.reshape(-1), minlength=40).tolist(), world, 512, max_share=0.1)
        assert max(parts) > 1                      # the Zipf head is split
        fused = ep_fused.FusedExpertParallelLayer(shard_owner, 512, 320, rank=rank, world=world,
                                                  rows_cap=2400, assignments_cap=(hi - lo) * 4,
                                                  exchange_groups=3, scheduler="dynamic_queue",
                                                  expert_parts=parts)
        for i in range(4):
            y = fused.forward(x[lo:hi].cuda(), ids[lo:hi].cuda(), w[fused.local_experts].cuda(),
                              topk_weights=gates.cuda() if i == 3 else None)
            if i == 2:
                same = same and torch.equal(y.view(torch.int16), want.view(torch.int16))
        fused.poll()
        same = same and torch.equal(y.cpu().view(torch.int16), want_z.view(torch.int16))
        dist.barrier()
        fused.close()
        # blocks of 8 rows and more travel as peer copies (copy engines), the rest as SM
        # stores; both kinds of flags gate the GEMM
        hosted = ep_fused.FusedExpertParallelLayer(owner, 512, 320, rank=rank, world=world,
                                                   rows_cap=2400, assignments_cap=(hi - lo) * 4,
                                                   exchange_groups=4, device_plan=False)
        planned = ep_fused.FusedExpertParallelLayer(owner, 512, 320, rank=rank, world=world,
                                                    rows_cap=2400, assignments_cap=(hi - lo) * 4,
                                                    exchange_groups=4)
        same = same and planned.device_plan and not hosted.device_plan
        for layer_ in (hosted, planned):
            for _ in range(3):
                y = layer_.forward(x[lo:hi].cuda(), ids[lo:hi].cuda(),
                                   w[layer_.local_experts].cuda())
            layer_.poll()
            same = same and torch.equal(y.view(torch.int16), want.view(torch.int16))
        same = same and hosted.last_local_m == planned.last_local_m
        dist.barrier()
        hosted.close()
        planned.close()
        once = ep_fused.FusedExpertParallelLayer(owner, 512, 320, rank=rank, world=world,
                                                 rows_cap=2400, assignments_cap=(hi - lo) * 4,
                                                 exchange_groups=4, send_once=True)
        once_hosted = ep_fused.FusedExpertParallelLayer(owner, 512, 320, rank=rank, world=world,
                                                        rows_cap=2400,
                                                        assignments_cap=(hi - lo) * 4,
                                                        exchange_groups=3, send_once=True,
                                                        device_plan=False, cta_group=1)
        for layer_ in (once, once_hosted):
            same = same and layer_.send_once
            for i in range(4):
                y = layer_.forward(x[lo:hi].cuda(), ids[lo:hi].cuda(),
                                   w[layer_.local_experts].cuda(),
                                   topk_weights=gates.cuda() if i == 3 else None)
                if i == 2:
                    same = same and torch.equal(y.view(torch.int16), want.view(torch.int16))
            layer_.poll()
            same = same and torch.equal(y.cpu().view(torch.int16), want_z.view(torch.int16))
        dist.barrier()
        once.close()
        once_hosted.close()
        copied = ep_fused.FusedExpertParallelLayer(owner, 512, 320, rank=rank, world=world,
                                                   rows_cap=2400, assignments_cap=(hi - lo) * 4,
                                                   exchange_groups=3, scheduler="dynamic_queue",
                                                   copy_engine_min_bytes=8 * 640)
        for i in range(4):
            y = copied.forward(x[lo:hi].cuda(), ids[lo:hi].cuda(), w[copied.local_experts].cuda(),
                               topk_weights=gates.cuda() if i == 3 else None)
            if i == 2:
                same = same and torch.equal(y.view(torch.int16), want.view(torch.int16))
                same = same and copied.copy_bytes > 0
        copied.poll()
        same = same and torch.equal(y.cpu().view(torch.int16), want_z.view(torch.int16))
        dist.barrier()
        copied.close()
        kept = ep_fused.FusedExpertParallelLayer(owner, 512, 320, rank=rank, world=world,
                                                 rows_cap=2400, assignments_cap=(hi - lo) * 4,
                                                 exchange_groups=2, push_results=False,
                                                 cta_group=1, bulk_copies=True,
                                                 copy_engine_min_bytes=0)
        for _ in range(2):
            y = kept.forward(x[lo:hi].cuda(), ids[lo:hi].cuda(), w[kept.local_experts].cuda())
        kept.poll()
        same = same and torch.equal(y.view(torch.int16), want.view(torch.int16))
        dist.barrier()
        kept.close()
        peer.close()
        Path(tmpdir, f"rank{rank}.txt").write_text(str(int(same)))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_nccl_ranks_equal_single_gpu_engine(engine, tmp_path):
    import torch
    import torch.multiprocessing as mp

    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_ep_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert Path(tmp_path, f"rank{r}.txt").read_text() == "1"
