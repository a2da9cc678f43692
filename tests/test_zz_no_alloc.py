"""bmoe_worklist_build_static: the worklist builder for callers that cannot
allocate device memory (fixed memory pools, plug-ins that are only handed
buffers). Its auxiliary arrays sit in a fixed array inside the library, so the
only buffers involved are the caller's counts (input) and tile records /
totals (outputs). Checked here against bmoe_worklist_build and against the CPU
oracle, record for record, on two calls in a row that share that array.
Collected last on purpose: a run that stops at the first failure has then
already run every other test."""

import ctypes as C

import numpy as np
import pytest

import support

pytestmark = pytest.mark.gpu


def build_static(engine, counts, n, tm, tn, order, raster, capacity):
    import torch

    cap = engine._capi
    c = torch.tensor(np.asarray(counts, dtype=np.int64), dtype=torch.int32, device="cuda")
    tiles = torch.full((max(1, capacity) * 20,), 0xEE, dtype=torch.uint8, device="cuda")
    totals = torch.zeros(8, dtype=torch.int32, device="cuda")
    req = cap.WorklistRequest(experts=len(counts), n=n, tile_m=tm, tile_n=tn, order=order,
                              raster=raster)
    rc = cap.load().bmoe_worklist_build_static(c.data_ptr(), C.byref(req), tiles.data_ptr(),
                                               capacity, totals.data_ptr(), None)
    return rc, tiles, totals


def build_existing(engine, counts, n, tm, tn, order, raster, capacity):
    import torch

    c = torch.tensor(np.asarray(counts, dtype=np.int64), dtype=torch.int32, device="cuda")
    tiles, ws, layout = engine.build_worklist_on_device(c, n, tm, tn, order=order, raster=raster,
                                                        tile_capacity=capacity)
    torch.cuda.synchronize()
    arrays = engine.read_worklist_arrays(ws, layout, len(counts))
    return tiles.cpu().numpy().view(support.TILE_DTYPE), arrays


def test_two_calls_in_a_row_match_the_workspace_entry_point(engine, oracle):
    import torch

    rng = np.random.default_rng(2026)
    # Second call has fewer experts and fewer tiles than the first, so leftovers
    # of the first call stay in the shared array while the second one runs.
    calls = [
        ((rng.integers(0, 900, size=1024) * (rng.random(1024) > 0.4)).astype(np.uint32),
         2048, 128, 256, 1, 1),
        ((rng.integers(0, 300, size=37) * (rng.random(37) > 0.2)).astype(np.uint32),
         520, 128, 128, 0, 0),
    ]
    for counts, n, tm, tn, order, raster in calls:
        want, arrays = build_existing(engine, counts, n, tm, tn, order, raster,
                                      len(support.engine_host_tiles(engine, counts, n, tm, tn)))
        total = arrays["total_tiles"]
        rc, tiles, totals = build_static(engine, counts, n, tm, tn, order, raster, total)
        assert rc == 0
        torch.cuda.synchronize()
        got = tiles.cpu().numpy().view(support.TILE_DTYPE)[:total]
        assert np.array_equal(got, want[:total])
        # and, directly, the CPU restatement of the reference's tile builder
        assert np.array_equal(got, oracle.build_tiles(counts, n, tm, tn, order=order,
                                                      raster=raster))
        t = totals.cpu().numpy().view(np.uint32)
        assert int(t[0]) == total and int(t[1]) == arrays["active_experts"]
        assert int(t[2]) | (int(t[3]) << 32) == arrays["total_rows"]
        assert int(t[4]) | (int(t[5]) << 32) == arrays["total_valid_elements"]
        assert int(t[6]) == 0


def test_sizes_beyond_the_fixed_array_are_rejected(engine):
    cap = engine._capi
    too_many = cap.WORKLIST_STATIC_MAX_EXPERTS + 1
    rc, _, _ = build_static(engine, [1] * too_many, 256, 128, 128, 0, 0, 16)
    assert rc == cap.INVALID_ARGUMENT
    rc, _, _ = build_static(engine, [1] * cap.WORKLIST_STATIC_MAX_EXPERTS, 256, 128, 128, 0, 0,
                            2 * cap.WORKLIST_STATIC_MAX_EXPERTS)
    assert rc == 0
