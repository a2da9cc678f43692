"""On-device worklist builder vs the host scheduler model: byte-for-byte."""

import numpy as np
import pytest

import support

pytestmark = pytest.mark.gpu


def device_tiles(engine, counts, n, tm, tn, order, raster, slack=3):
    import torch

    c = torch.tensor(np.asarray(counts, dtype=np.int64), dtype=torch.int32, device="cuda")
    want = support.engine_host_tiles(engine, counts, n, tm, tn, order=order, raster=raster)
    cap = len(want) + slack
    tiles, ws, layout = engine.build_worklist_on_device(c, n, tm, tn, order=order, raster=raster,
                                                        tile_capacity=cap)
    torch.cuda.synchronize()
    got = tiles.cpu().numpy().view(support.TILE_DTYPE)[: len(want)]
    return got, want, engine.read_worklist_arrays(ws, layout, len(counts))


def check_arrays(arrays, counts, n, tm, tn, want_tiles, order, oracle):
    counts = np.asarray(counts, dtype=np.uint64)
    e = len(counts)
    m_tiles = (counts + tm - 1) // tm
    n_tiles = (n + tn - 1) // tn
    assert arrays["total_tiles"] == len(want_tiles) and arrays["overflow"] == 0
    assert arrays["active_experts"] == int((counts > 0).sum())
    assert arrays["total_rows"] == int(counts.sum())
    assert arrays["total_valid_elements"] == int(counts.sum()) * n
    assert np.array_equal(arrays["expert_m_tiles"], m_tiles.astype(np.uint32))
    assert np.array_equal(arrays["expert_tiles"], (m_tiles * n_tiles).astype(np.uint32))
    assert np.array_equal(arrays["row_offsets"], np.concatenate([[0], np.cumsum(counts)]))
    assert np.array_equal(arrays["tile_offsets"],
                          np.concatenate([[0], np.cumsum(m_tiles * n_tiles)]).astype(np.uint32))
    active = np.flatnonzero(counts > 0).astype(np.uint32)
    assert np.array_equal(arrays["active_ids"][: len(active)], active)
    assert np.all(arrays["active_ids"][len(active):] == 0xFFFFFFFF)
    # visiting order: identity, or stable descending by tile count
    if order == 0:
        assert np.array_equal(arrays["visit_order"], np.arange(e, dtype=np.uint32))
    else:
        key = (m_tiles * n_tiles).astype(np.int64)
        assert np.array_equal(arrays["visit_order"],
                              np.argsort(-key, kind="stable").astype(np.uint32))
    visit_tiles = (m_tiles * n_tiles)[arrays["visit_order"]]
    assert np.array_equal(arrays["visit_tile_offsets"],
                          np.concatenate([[0], np.cumsum(visit_tiles)]).astype(np.uint32))


def test_reference_unit_case_and_edges(engine, oracle, golden):
    for case in golden["tile_cases"]:
        if sum(case["counts"]) == 0:
            continue
        for order in (0, 1):
            got, want, arrays = device_tiles(engine, case["counts"], case["n"], case["tile_m"],
                                             case["tile_n"], order, 0)
            assert [list(map(int, t)) for t in got.tolist()] == case[f"order{order}"]
            check_arrays(arrays, case["counts"], case["n"], case["tile_m"], case["tile_n"], want,
                         order, oracle)


def test_all_inactive_builds_an_empty_worklist(engine, oracle):
    got, want, arrays = device_tiles(engine, [0, 0, 0, 0], 256, 128, 128, 0, 0)
    assert len(want) == 0 and arrays["total_tiles"] == 0 and arrays["active_experts"] == 0
    assert np.all(arrays["active_ids"] == 0xFFFFFFFF)


def test_benchmark_workloads_bit_exact(engine, golden):
    for name, entry in golden["workloads"].items():
        n, tm, _ = entry["shape"]
        for tn in (128, 256):
            for order in (0, 1):
                got, want, _ = device_tiles(engine, entry["counts"], n, tm, tn, order, 0)
                assert support.sha(got) == entry[f"tiles_sha256_tn{tn}_order{order}"], (name, tn, order)
                alt, want_alt, _ = device_tiles(engine, entry["counts"], n, tm, tn, order, 1)
                assert np.array_equal(alt, want_alt)


def test_randomised_against_oracle(engine, oracle):
    rng = np.random.default_rng(99)
    for trial in range(40):
        e = int(rng.choice([1, 2, 7, 33, 257, 1024, 1500, 3000]))
        zero_p = float(rng.choice([0.0, 0.3, 0.9]))
        counts = (rng.integers(0, 600, size=e) * (rng.random(e) >= zero_p)).astype(np.uint32)
        if counts.sum() == 0:
            counts[rng.integers(0, e)] = 5
        n = int(rng.integers(1, 2100))
        tm = int(rng.choice([64, 128, 256]))
        tn = int(rng.choice([64, 128, 256]))
        order, raster = int(rng.integers(0, 2)), int(rng.integers(0, 2))
        got, want, arrays = device_tiles(engine, counts, n, tm, tn, order, raster)
        assert np.array_equal(got, want), (trial, e, n, tm, tn, order, raster)
        assert np.array_equal(want, oracle.build_tiles(counts, n, tm, tn, order=order, raster=raster))
        check_arrays(arrays, counts, n, tm, tn, want, order, oracle)


def test_capacity_overflow_is_flagged_not_written(engine):
    import torch

    counts = [300, 300]
    c = torch.tensor(counts, dtype=torch.int32, device="cuda")
    want = support.engine_host_tiles(engine, counts, 512, 128, 128)
    cap = len(want) - 5
    tiles, ws, layout = engine.build_worklist_on_device(c, 512, 128, 128, tile_capacity=cap)
    guard = tiles.clone()
    torch.cuda.synchronize()
    arrays = engine.read_worklist_arrays(ws, layout, 2)
    assert arrays["overflow"] == 1 and arrays["total_tiles"] == len(want)
    got = tiles.cpu().numpy().view(support.TILE_DTYPE)
    assert len(got) == cap and np.array_equal(got, want[:cap])
    assert guard.numel() == cap * 20
