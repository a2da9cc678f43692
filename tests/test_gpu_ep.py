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
    finally:
        layer.close()


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
        from bmoe_b200 import ep_peer

        peer = ep_peer.PeerExpertParallelLayer(owner, 512, 320, rank=rank, world=world,
                                               rows_cap=2400, scheduler="clc")
        for _ in range(3):
            y = peer.forward(x[lo:hi].cuda(), ids[lo:hi].cuda(), w[peer.local_experts].cuda())
        peer.poll()
        same = same and torch.equal(y.view(torch.int16), want.view(torch.int16))
        dist.barrier()
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
