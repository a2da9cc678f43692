"""Pins the CPU oracle: against the reference's own compiled sources where they
were built (oracle/_ref), and against the committed fixtures generated from the
reference (tests/golden/reference_vectors.json)."""

import numpy as np
import pytest

import support


def _gen_args(cfg):
    return dict(experts=cfg["experts"], total_tokens=cfg["total_tokens"],
                distribution=cfg["distribution"], seed=cfg["seed"],
                zipf_alpha=cfg["zipf_alpha"], heavy_fraction=cfg["heavy_fraction"],
                heavy_share=cfg["heavy_share"], inactive_fraction=cfg["inactive_fraction"])


def test_generator_matches_golden_counts(oracle, golden):
    for name, entry in golden["workloads"].items():
        rc, counts = oracle.generate_counts(**_gen_args(entry["config"]))
        assert rc == 0
        assert counts.tolist() == entry["counts"], name


def test_workload_metrics_match_golden_bit_for_bit(oracle, golden):
    for name, entry in golden["workloads"].items():
        n, tm, tn = entry["shape"]
        rc, reals, ints = oracle.workload_metrics(entry["counts"], n, tm, tn)
        assert rc == 0
        assert [float(x).hex() for x in reals] == entry["metrics"], name
        assert int(ints[0]) == entry["active_experts"] and int(ints[1]) == entry["total_tiles"]


def test_tiles_match_golden_hashes(oracle, golden):
    for name, entry in golden["workloads"].items():
        n, tm, _ = entry["shape"]
        for tn in (128, 256):
            for order in (0, 1):
                tiles = oracle.build_tiles(entry["counts"], n, tm, tn, order=order)
                assert len(tiles) == entry[f"tiles_count_tn{tn}"]
                assert support.sha(tiles) == entry[f"tiles_sha256_tn{tn}_order{order}"], (name, tn, order)


def test_schedules_match_golden(oracle, golden):
    for name, entry in golden["workloads"].items():
        n, tm, tn = entry["shape"]
        for sched, want in entry["schedule_148"].items():
            tiles, offs, ints, reals = oracle.simulate(int(sched), entry["counts"], n, tm, tn, 148)
            assert support.sha(tiles) == want["tiles_sha256"], (name, sched)
            assert support.sha(offs) == want["offsets_sha256"], (name, sched)
            assert [int(x) for x in ints] == want["ints"], (name, sched)
            assert [float(x).hex() for x in reals] == want["reals"], (name, sched)


def test_small_tile_cases_record_for_record(oracle, golden):
    for case in golden["tile_cases"]:
        for order in (0, 1):
            tiles = oracle.build_tiles(case["counts"], case["n"], case["tile_m"], case["tile_n"],
                                       order=order)
            assert [list(map(int, t)) for t in tiles.tolist()] == case[f"order{order}"]
        for sched in range(5):
            want = case[f"sched{sched}_cta3"]
            tiles, offs, ints, reals = oracle.simulate(sched, case["counts"], case["n"],
                                                       case["tile_m"], case["tile_n"], 3)
            assert [list(map(int, t)) for t in tiles.tolist()] == want["tiles"]
            assert [int(x) for x in offs] == want["offsets"]
            assert [int(x) for x in ints] == want["ints"]
            assert [float(x).hex() for x in reals] == want["reals"]


def test_dispatch_matches_reference_python(oracle, golden):
    order = ["mean_m", "cv_m", "max_over_mean_m", "inactive_expert_ratio", "small_m_expert_ratio",
             "expert_tile_cv", "max_expert_tiles_over_mean", "tiles_per_cta", "useful_work_ratio"]
    variants = ["v0_nonpersistent", "v1_static_ws", "v2_dynamic", "v3_chunked", "v4_hybrid"]
    for case in golden["planner"]["feature_cases"]:
        spec = case["spec"]
        rc, out, tiles = oracle.routing_features(case["counts"], spec["n"], 128, 128,
                                                 spec.get("cta_count", 148))
        assert rc == 0
        assert tiles == case["features"]["active_tiles"] == case["tile_count"]
        assert [float(x).hex() for x in out] == [case["features"][k] for k in order], spec
        pick = oracle.select_variant(out[7], out[1], out[3])
        assert variants[pick] == case["select_kernel"]


def test_gemm_oracle_reproduces_reference_known_answers(oracle, golden):
    """The KAT inputs have exact FP32 sums, so the BF16 result is fixed by
    arithmetic; the oracle must hit it bit for bit, and its FP32 and FP64
    accumulations must agree exactly there."""
    for name, want in golden["gemm_kats"].items():
        counts, n, k, a_bits, w_bits = support.kat_inputs(name)
        assert counts == want["counts"] and n == want["n"] and k == want["k"]
        out = oracle.grouped_gemm(a_bits, w_bits, counts, n, k, want_f32=True, want_f64=True)
        bits = out["bf16"].reshape(-1)
        assert bits.size == want["d_elems"]
        assert bits[:16].tolist() == want["d_first16"]
        assert support.sha(bits) == want["d_sha256"], name
        assert np.array_equal(out["f32"].astype(np.float64), out["f64"])


def test_gemm_oracle_matches_torch_expression(oracle):
    """Reference check expression (python/blackwell_moe_tirx/runner.py:222-224):
    A.float() @ B.float().T rounded to BF16; agreement within 1 BF16 ulp of the
    reference's own tolerance (the summation order differs)."""
    torch = pytest.importorskip("torch")
    gen = torch.Generator().manual_seed(5)
    counts = [33, 0, 130]
    n, k = 96, 256
    a = torch.randn(sum(counts), k, generator=gen).to(torch.bfloat16)
    w = (torch.randn(len(counts), n, k, generator=gen) * k ** -0.5).to(torch.bfloat16)
    out = oracle.grouped_gemm(a.view(torch.int16).numpy().view(np.uint16),
                              w.view(torch.int16).numpy().view(np.uint16), counts, n, k,
                              want_f64=True)
    got = support.bf16_bits_to_f32(out["bf16"])
    row = 0
    for e, m in enumerate(counts):
        if m == 0:
            continue
        want = (a[row:row + m].float() @ w[e].float().T).to(torch.bfloat16).float().numpy()
        assert np.allclose(got[row:row + m], want, rtol=2e-2, atol=5e-2)
        ulp = np.maximum(np.abs(want), 2.0 ** -6) * 2.0 ** -7
        assert np.all(np.abs(got[row:row + m] - want) <= ulp)
        row += m
    # sampled rows leave the others untouched
    part = oracle.grouped_gemm(a.view(torch.int16).numpy().view(np.uint16),
                               w.view(torch.int16).numpy().view(np.uint16), counts, n, k,
                               row_stride=4, row_phase=1)
    assert part["rows"] == sum(len(range(1, m, 4)) for m in counts)
    assert np.array_equal(part["bf16"][1], out["bf16"][1]) and not part["bf16"][0].any()


def test_probe_checksum_is_deterministic_and_tile_specific(oracle):
    a = oracle.probe_checksum((3, 1, 2, 128, 128), 2)
    assert a == oracle.probe_checksum((3, 1, 2, 128, 128), 2)
    assert a != oracle.probe_checksum((3, 1, 3, 128, 128), 2)
    assert a != oracle.probe_checksum((3, 1, 2, 128, 128), 1)


# ---- against the reference's own compiled host sources (built in place) ----

def test_oracle_equals_compiled_reference_generator(oracle, reflib):
    rng = np.random.default_rng(11)
    for dist in range(4):
        for _ in range(6):
            e = int(rng.integers(1, 300))
            t = int(rng.integers(0, 50000))
            kw = dict(seed=int(rng.integers(0, 2**40)), zipf_alpha=float(rng.uniform(0.1, 2.5)),
                      heavy_fraction=float(rng.uniform(0.01, 1.0)),
                      heavy_share=float(rng.uniform(0, 1)),
                      inactive_fraction=float(rng.uniform(0, 1)))
            rc_o, c_o = oracle.generate_counts(e, t, dist, **kw)
            rc_r, c_r = reflib.generate_counts(e, t, dist, **kw)
            assert rc_o == rc_r == 0
            assert np.array_equal(c_o, c_r), (dist, e, t, kw)
    # rejected configurations are rejected by both
    for kw in (dict(zipf_alpha=0.0), dict(heavy_fraction=0.0), dict(heavy_share=1.5),
               dict(inactive_fraction=-0.1)):
        assert oracle.generate_counts(8, 100, 3, **kw)[0] == -1
        assert reflib.generate_counts(8, 100, 3, **kw)[0] == -1
    assert oracle.generate_counts(0, 100, 0)[0] == -1 and reflib.generate_counts(0, 100, 0)[0] == -1


def test_oracle_equals_compiled_reference_scheduler(oracle, reflib):
    rng = np.random.default_rng(3)
    for _ in range(40):
        e = int(rng.integers(1, 60))
        counts = (rng.integers(0, 900, size=e) * (rng.random(e) > 0.25)).astype(np.uint32)
        n = int(rng.integers(1, 3000))
        tm = int(rng.choice([32, 64, 128, 256]))
        tn = int(rng.choice([64, 128, 256, 96]))
        for order in (0, 1):
            assert np.array_equal(oracle.build_tiles(counts, n, tm, tn, order=order),
                                  reflib.build_tiles(counts, n, tm, tn, order=order))
        ctas = int(rng.integers(1, 160))
        for sched in range(5):
            o = oracle.simulate(sched, counts, n, tm, tn, ctas)
            r = reflib.simulate(sched, counts, n, tm, tn, ctas)
            assert np.array_equal(o[0], r[0]) and np.array_equal(o[1], r[1])
            assert np.array_equal(o[2], r[2])
            assert [float(x).hex() for x in o[3]] == [float(x).hex() for x in r[3]]
        mo, mr = oracle.workload_metrics(counts, n, tm, tn), reflib.workload_metrics(counts, n, tm, tn)
        assert [float(x).hex() for x in mo[1]] == [float(x).hex() for x in mr[1]]
        assert np.array_equal(mo[2], mr[2])


def test_combine_topk_definition(oracle):
    """The weighted top-k combine has no reference counterpart; this pins the CPU
    statement of the step itself: FP32, terms in ascending j, one BF16 rounding,
    dropped (negative) rows skipped. Weights are multiples of 1/8 so that every
    product is exact in FP32 and a plain float32 loop is the same arithmetic."""
    rng = np.random.default_rng(7)
    src = support.f32_to_bf16_bits(rng.standard_normal((40, 24)).astype(np.float32))
    rows = rng.integers(0, 40, size=(9, 3)).astype(np.int64)
    rows[2, 1] = -1
    rows[5, :] = -1
    weights = (rng.integers(-8, 9, size=(9, 3)) / 8.0).astype(np.float32)
    got = oracle.combine_topk(src, rows, weights)
    vals = support.bf16_bits_to_f32(src)
    want = np.zeros((9, 24), dtype=np.float32)
    for t in range(9):
        for j in range(3):
            if rows[t, j] >= 0:
                want[t] = (want[t] + weights[t, j] * vals[rows[t, j]]).astype(np.float32)
    assert np.array_equal(got, support.f32_to_bf16_bits(want))
    assert not got[5].any()
    ones = oracle.combine_topk(src, rows, None)
    assert np.array_equal(ones, oracle.combine_topk(src, rows, np.ones_like(weights)))


def test_e4m3_codec_equals_torch_float8(oracle):
    """The oracle's FP8 E4M3 decode and encode against an independent implementation,
    torch.float8_e4m3fn on the CPU: all 256 codes decode to the same value (the two NaN
    codes to NaN), every decoded value is a BF16 value, and round-to-nearest-even encoding
    of values inside the finite range (normals, subnormals, exact ties, +-0) gives the same
    code. Beyond +-448 the oracle saturates to the largest finite code."""
    import torch

    codes = np.arange(256, dtype=np.uint8)
    want = torch.from_numpy(codes.copy()).view(torch.float8_e4m3fn).to(torch.float32).numpy()
    as_bf16 = support.bf16_bits_to_f32(oracle.e4m3_to_bf16(codes))
    nan = np.isnan(want)
    assert list(np.flatnonzero(nan)) == [0x7F, 0xFF]
    assert np.array_equal(np.isnan(as_bf16), nan)
    assert np.array_equal(as_bf16[~nan].view(np.uint32), want[~nan].view(np.uint32))

    rng = np.random.default_rng(5)
    finite = want[~nan]
    ties = (np.sort(finite)[:-1] + np.sort(finite)[1:]) / 2.0          # exact midpoints
    values = np.concatenate([
        finite, ties.astype(np.float32), rng.normal(0, 1, 4000).astype(np.float32),
        rng.normal(0, 0.01, 2000).astype(np.float32), rng.uniform(-448, 448, 2000).astype(
            np.float32), np.array([0.0, -0.0, 2.0 ** -10, -(2.0 ** -10), 448.0, -448.0],
                                  dtype=np.float32)])
    mine = oracle.f32_to_e4m3(values)
    theirs = torch.from_numpy(values).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    assert np.array_equal(mine, theirs)
    assert list(oracle.f32_to_e4m3(np.array([1e6, -1e6, 460.0], dtype=np.float32))) == [
        0x7E, 0xFE, 0x7E]
