"""Scheduler probe on the GPU: exact-once coverage, per-CTA tallies and the
per-tile checksum (expectations of the reference's tests/test_scheduler_probe.cu:100-128)."""

import numpy as np
import pytest

import support

pytestmark = pytest.mark.gpu


def synthetic_tiles():
    rec = np.zeros(37, dtype=support.TILE_DTYPE)
    for i in range(37):
        rec[i] = (i % 7, i // 7, i % 4, 17 if i % 5 == 0 else 128, 65 if i % 3 == 0 else 128)
    return rec


def run_probe(engine, scheduler, tiles, ctas, claim, work_scale=2):
    import torch

    t = torch.from_numpy(tiles.view(np.uint8).copy()).cuda()
    n = len(tiles)
    nxt = torch.zeros(1, dtype=torch.int32, device="cuda")
    visits = torch.zeros(n, dtype=torch.int32, device="cuda")
    sums = torch.zeros(n, dtype=torch.int64, device="cuda")
    cta_tiles = torch.zeros(ctas, dtype=torch.int32, device="cuda")
    cta_work = torch.zeros(ctas, dtype=torch.int64, device="cuda")
    rc = engine.launch_scheduler_probe(scheduler, t, n, ctas, claim_size=claim,
                                       work_scale=work_scale, next_tile=nxt, tile_visits=visits,
                                       tile_checksums=sums, cta_tile_counts=cta_tiles,
                                       cta_valid_elements=cta_work)
    assert rc == 0
    torch.cuda.synchronize()
    return (visits.cpu().numpy(), sums.cpu().numpy().view(np.uint64), cta_tiles.cpu().numpy(),
            cta_work.cpu().numpy(), int(nxt.item()))


@pytest.mark.parametrize("scheduler,claim", [(0, 1), (1, 1), (1, 4)])
def test_reference_probe_case(engine, oracle, scheduler, claim):
    tiles = synthetic_tiles()
    visits, sums, cta_tiles, cta_work, head = run_probe(engine, scheduler, tiles, 8, claim)
    assert np.all(visits == 1)
    assert int(cta_tiles.sum()) == len(tiles)
    assert int(cta_work.sum()) == int((tiles["valid_m"].astype(np.int64) * tiles["valid_n"]).sum())
    want = np.array([oracle.probe_checksum(tuple(t), 2) for t in tiles.tolist()], dtype=np.uint64)
    assert np.array_equal(sums, want)
    if scheduler == 0:
        # grid stride: CTA c runs tiles c, c + 8, ...
        assert cta_tiles.tolist() == [len(range(c, 37, 8)) for c in range(8)]
    else:
        # every CTA's failing last claim also advances the head
        assert head >= len(tiles) and (head - 0) % claim == 0


def test_probe_on_a_benchmark_worklist(engine, oracle, golden):
    counts = golden["workloads"]["c4_zipf15_e128"]["counts"]
    tiles = support.engine_host_tiles(engine, counts, 768, 128, 128)
    for scheduler, claim in ((0, 1), (1, 1), (1, 8)):
        visits, sums, cta_tiles, cta_work, _ = run_probe(engine, scheduler, tiles, 148, claim, 1)
        assert np.all(visits == 1) and int(cta_tiles.sum()) == len(tiles)
        assert int(cta_work.sum()) == int(sum(counts)) * 768
        pick = np.random.default_rng(0).integers(0, len(tiles), size=64)
        for i in pick:
            assert int(sums[i]) == oracle.probe_checksum(tuple(tiles[i].tolist()), 1)


def test_probe_argument_checks(engine):
    import torch

    t = torch.zeros(20, dtype=torch.uint8, device="cuda")
    assert engine.launch_scheduler_probe(0, t, 1, 1) == engine._capi.INVALID_ARGUMENT
    assert engine.launch_scheduler_probe(7, t, 1, 1) == engine._capi.INVALID_ARGUMENT
