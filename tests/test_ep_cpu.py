"""Expert-parallel layer on CPU ranks (gloo, world_size 2 and 3): placement, split
sizes and the permutation round trip. The device operations are injected (row
gather = index_select, grouped GEMM = the CPU oracle), so no GPU is needed; the
result must equal the single-process oracle GEMM bit for bit."""

import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


class OracleOps:
    """CPU stand-ins for the layer's device operations (test infrastructure)."""

    def __init__(self):
        import support

        self.oracle = support.Oracle()
        self.launches = 0

    def gather_rows(self, src, index, out=None):
        return src.index_select(0, index)

    def combine_topk(self, src, rows, weights=None, out=None):
        import torch

        bits = self.oracle.combine_topk(
            src.contiguous().view(torch.int16).numpy().view(np.uint16), rows.numpy(),
            None if weights is None else weights.numpy())
        return torch.from_numpy(bits.view(np.int16).copy()).view(torch.bfloat16)

    def grouped_gemm(self, a, w, counts, out=None, slot=0):
        import torch

        n, k = int(w.shape[1]), int(w.shape[2])
        if sum(counts) == 0:
            return torch.empty(0, n, dtype=torch.bfloat16)
        bits = self.oracle.grouped_gemm(
            a.contiguous().view(torch.int16).numpy().view(np.uint16),
            w.contiguous().view(torch.int16).numpy().view(np.uint16), counts, n, k)["bf16"]
        return torch.from_numpy(bits.view(np.int16).copy()).view(torch.bfloat16)


def worker(rank, world, port, tmpdir, groups=1):
    for p in (ROOT, ROOT / "tests", ROOT / "oracle"):
        sys.path.insert(0, str(p))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import torch
    import torch.distributed as dist

    import bmoe_b200
    from bmoe_b200 import ep

    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        experts, top_k, tokens, n, k = 12, 2, 96, 64, 40
        gen = torch.Generator().manual_seed(2026)
        # identical on every rank: global routing, inputs and weights
        probs = 1.0 / torch.arange(1, experts + 1, dtype=torch.float64)
        probs[5] = 0.0  # an expert nobody routes to
        ids_all = torch.multinomial(probs.expand(tokens, -1), top_k, replacement=False,
                                    generator=gen)
        x_all = torch.randn(tokens, k, generator=gen).to(torch.bfloat16)
        w_all = (torch.randn(experts, n, k, generator=gen) * k ** -0.5).to(torch.bfloat16)
        global_counts = torch.bincount(ids_all.reshape(-1), minlength=experts).tolist()
        owner, loads = ep.place_experts(global_counts, world, n, tile_m=128, tile_n=128)
        assert sorted(set(owner)) == list(range(world)) and sum(loads) == sum(
            (c + 127) // 128 for c in global_counts)
        # uneven token split across ranks
        bounds = [0] + [tokens * (r + 1) // world + (3 if r == 0 else 0) for r in range(world)]
        bounds[-1] = tokens
        lo, hi = bounds[rank], bounds[rank + 1]
        layer = ep.ExpertParallelLayer(owner, n, k, rank=rank, world=world, ops=OracleOps(),
                                       pipeline_groups=groups)
        w_local = w_all[layer.local_experts]
        y = layer.forward(x_all[lo:hi], ids_all[lo:hi], w_local)

        # single-process reference: every assignment through the oracle GEMM
        order = torch.sort(ids_all.reshape(-1), stable=True).indices
        a_ref = x_all[order // top_k]
        d_ref = OracleOps().grouped_gemm(a_ref, w_all, global_counts)
        y_ref = torch.empty_like(d_ref)
        y_ref[order] = d_ref
        want = y_ref[lo * top_k:hi * top_k]
        same = torch.equal(y.view(torch.int16), want.view(torch.int16))
        if groups == 1:
            # weighted top-k combine as the last step: equals the combine of the rows
            gates = torch.rand(tokens, top_k, generator=gen)
            z = layer.forward(x_all[lo:hi], ids_all[lo:hi], w_local, topk_weights=gates[lo:hi])
            rows = torch.arange((hi - lo) * top_k).reshape(-1, top_k)
            z_ref = OracleOps().combine_topk(want, rows, gates[lo:hi])
            same = same and z.shape == (hi - lo, n) and torch.equal(
                z.view(torch.int16), z_ref.view(torch.int16))
        Path(tmpdir, f"rank{rank}.txt").write_text(
            f"{int(same)} {y.shape[0]} {sum(layer.last_local_m)}")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,groups", [(2, 1), (3, 1), (2, 3), (3, 2)])
def test_ep_round_trip_equals_single_process(world, groups, tmp_path, engine):
    import torch.multiprocessing as mp

    mp.spawn(worker, args=(world, free_port(), str(tmp_path), groups), nprocs=world, join=True)
    rows = 0
    for r in range(world):
        same, count, local = Path(tmp_path, f"rank{r}.txt").read_text().split()
        assert same == "1", f"rank {r} output differs from the single-process result"
        rows += int(local)
    assert rows == 96 * 2  # every assignment computed by exactly one owner


def test_placement_is_deterministic_lpt(engine):
    from bmoe_b200 import ep

    counts = [1000, 10, 0, 500, 500, 129, 128, 1]
    owner, loads = ep.place_experts(counts, 3, 256, tile_m=128, tile_n=128)
    # tiles (x2 column tiles): 16, 2, 0, 8, 8, 4, 2, 2 -> order e0, e3, e4, e5, e1, e6, e7, e2
    assert owner == [0, 2, 2, 1, 2, 1, 2, 1]
    assert loads == [16, 14, 12]
    assert ep.place_experts(counts, 3, 256, tile_m=128, tile_n=128) == (owner, loads)
    capped, _ = ep.place_experts(counts, 4, 256, tile_m=128, tile_n=128, max_experts_per_rank=2)
    assert all(capped.count(r) == 2 for r in range(4))
    with pytest.raises(Exception):
        ep.place_experts(counts, 3, 256, max_experts_per_rank=2)  # 6 slots for 8 experts


def test_peer_route_plan_builds_the_single_gpu_packing(engine):
    """plan_routes() (index arithmetic of the peer-memory exchange) on simulated
    ranks: every owner's buffer is written exactly once per row, expert-major, and
    inside an expert in global assignment order - the single-GPU packing."""
    import torch

    from bmoe_b200 import ep, ep_peer

    gen = torch.Generator().manual_seed(9)
    world, experts, top_k, tokens = 3, 10, 2, 50
    probs = torch.rand(experts, generator=gen) + 0.05
    probs[4] = 0.0
    ids_all = torch.multinomial(probs.expand(tokens, -1), top_k, replacement=False, generator=gen)
    counts = torch.bincount(ids_all.reshape(-1), minlength=experts).tolist()
    owner, _ = ep.place_experts(counts, world, 256, tile_m=128, tile_n=128)
    bounds = [0, 13, 31, tokens]
    counts_all = torch.stack([
        torch.bincount(ids_all[bounds[r]:bounds[r + 1]].reshape(-1), minlength=experts)
        for r in range(world)]).to(torch.int64)
    # global assignment id written into the owner's buffer slot
    buffers = [dict() for _ in range(world)]
    for r in range(world):
        flat = ids_all[bounds[r]:bounds[r + 1]].reshape(-1)
        perm, src_token, dst_rank, dst_row = ep_peer.plan_routes(counts_all, owner, r, flat, top_k)
        assert torch.equal(src_token, perm // top_k)
        for i in range(perm.numel()):
            slot = buffers[int(dst_rank[i])]
            assert int(dst_row[i]) not in slot, "two assignments routed to one row"
            slot[int(dst_row[i])] = bounds[r] * top_k + int(perm[i])
    flat_all = ids_all.reshape(-1)
    for r in range(world):
        mine = [e for e in range(experts) if owner[e] == r]
        want = [j for e in mine for j in range(flat_all.numel()) if int(flat_all[j]) == e]
        got = [buffers[r][row] for row in range(len(buffers[r]))]
        assert sorted(buffers[r]) == list(range(len(want)))
        assert got == want


def test_fused_exchange_step_tables_cover_every_owner_buffer_once(engine):
    """plan_step() of the overlapped exchange: with the cursor of the dispatch kernel
    emulated in assignment order, the rows of all sources fill every owner's packed
    buffer exactly once, expert-major in ascending id, and the expert groups are
    contiguous runs of an owner's experts in packed order."""
    import torch

    from bmoe_b200 import ep, ep_fused

    gen = torch.Generator().manual_seed(21)
    world, experts, top_k, tokens, groups = 3, 14, 2, 120, 4
    probs = torch.rand(experts, generator=gen) + 0.05
    probs[6] = 0.0
    ids_all = torch.multinomial(probs.expand(tokens, -1), top_k, replacement=False, generator=gen)
    global_counts = torch.bincount(ids_all.reshape(-1), minlength=experts)
    owner, _ = ep.place_experts(global_counts.tolist(), world, 256)
    bounds = [0, 37, 90, tokens]
    counts_all = np.stack([
        np.bincount(ids_all[bounds[r]:bounds[r + 1]].reshape(-1).numpy(), minlength=experts)
        for r in range(world)]).astype(np.int64)
    steps = [ep_fused.plan_step(counts_all, owner, r, groups, tile_m=16) for r in range(world)]
    for r in range(world):
        assert steps[r]["local_experts"] == [e for e in range(experts) if owner[e] == r]
        assert steps[r]["local_m"] == [int(global_counts[e]) for e in steps[r]["local_experts"]]
        assert np.array_equal(steps[r]["group_of"], steps[0]["group_of"])   # same on every rank
        g_local = steps[r]["group_local"]
        assert np.all(np.diff(g_local.astype(np.int64)) >= 0) and g_local.max(initial=0) < groups
    filled = [np.full(steps[q]["total_local"], -1, dtype=np.int64) for q in range(world)]
    for r in range(world):
        cursor = np.zeros(experts, dtype=np.int64)
        flat = ids_all[bounds[r]:bounds[r + 1]].reshape(-1).numpy()
        # route entries per bucket: exchange groups of rows that leave, then rows that stay
        sizes = np.zeros(groups + 2, dtype=np.int64)     # the last bucket: copy-engine blocks
        for e in flat:
            sizes[groups if owner[e] == r else steps[r]["group_of"][e]] += 1
        assert np.array_equal(np.diff(steps[r]["bucket_offset"].astype(np.int64)), sizes)
        assert steps[r]["bucket_offset"][-1] == flat.size
        for e in flat:
            row = steps[r]["row_base"][e] + cursor[e]
            cursor[e] += 1
            assert filled[owner[e]][row] == -1, "two assignments share a row"
            filled[owner[e]][row] = e
    for q in range(world):
        want = np.repeat(steps[q]["local_experts"], steps[q]["local_m"])
        assert np.array_equal(filled[q], want)


def test_copy_engine_blocks_are_agreed_on_by_sender_and_receiver(engine):
    """Blocks of at least copy_min_rows rows leave as peer copies: the sender's list, its
    staging layout and bucket sizes, and every receiver's per-group source mask follow from
    the same count matrix and must describe the same set of blocks."""
    from bmoe_b200 import ep_fused

    rng = np.random.default_rng(5)
    world, experts, groups, min_rows = 4, 23, 3, 120
    counts_all = (rng.integers(0, 400, size=(world, experts)) *
                  (rng.random((world, experts)) > 0.2)).astype(np.int64)
    owner = [int(x) for x in rng.integers(0, world, size=experts)]
    steps = [ep_fused.plan_step(counts_all, owner, r, groups, tile_m=64, copy_min_rows=min_rows)
             for r in range(world)]
    none = [ep_fused.plan_step(counts_all, owner, r, groups, tile_m=64) for r in range(world)]
    masks = np.zeros((world, groups), dtype=np.uint32)
    for r in range(world):
        st = steps[r]
        want = [e for e in range(experts) if owner[e] != r and counts_all[r][e] >= min_rows]
        assert sorted(st["copy_experts"].tolist()) == want
        assert none[r]["copy_experts"].size == 0 and not none[r]["copy_mask"].any()
        assert np.array_equal(st["row_base"], none[r]["row_base"])       # placement unchanged
        # sending order: by (group, owner, id); staging rows back to back in that order
        keys = [(int(st["group_of"][e]), owner[e], int(e)) for e in st["copy_experts"]]
        assert keys == sorted(keys)
        at = 0
        for e in st["copy_experts"]:
            assert st["staging_row_base"][e] == at
            at += counts_all[r][e]
        assert all(st["staging_row_base"][e] == -1 for e in range(experts) if e not in want)
        sizes = np.diff(st["bucket_offset"].astype(np.int64))
        assert sizes[groups + 1] == at and sizes.sum() == counts_all[r].sum()
        assert sizes[groups] == sum(counts_all[r][e] for e in range(experts) if owner[e] == r)
        for e in want:
            masks[owner[e], st["group_of"][e]] |= np.uint32(1 << r)
    for q in range(world):
        assert np.array_equal(steps[q]["copy_mask"], masks[q]), q


def test_hot_experts_are_split_into_row_shards(engine):
    from bmoe_b200 import ep

    counts = [4000, 300, 300, 200, 100, 100, 0, 50]
    parts, shard_owner, loads = ep.split_and_place_experts(counts, 4, 256, tile_m=128, tile_n=256)
    # tiles: 32 3 3 2 1 1 0 1 -> 43, fair share 10.75, shards of at most 5 tiles
    assert parts == [4, 1, 1, 1, 1, 1, 1, 1]       # capped at one shard per rank
    assert len(shard_owner) == sum(parts) and sorted(set(shard_owner[:4])) == [0, 1, 2, 3]
    assert sum(loads) == 4 * 8 + 11 and max(loads) - min(loads) <= 3
    whole, owner, _ = ep.split_and_place_experts(counts, 1, 256)
    assert whole == [1] * 8 and owner == [0] * 8
