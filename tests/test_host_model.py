"""Host side of the product (C++ library through the C interface, and the Python
planner over it) against the oracle, the golden fixtures and the reference's
own unit-test expectations (tests/test_workload.cpp, tests/test_scheduler.cpp,
tests/test_tirx_worklist.py)."""

import ctypes as C

import numpy as np
import pytest

import support


def gen_counts(engine, experts, total, dist, **kw):
    cap = engine._capi
    cfg = cap.WorkloadConfig(experts=experts, distribution=dist, total_tokens=total,
                             seed=kw.get("seed", 2026), zipf_alpha=kw.get("zipf_alpha", 1.2),
                             heavy_hitter_fraction=kw.get("heavy_fraction", 0.1),
                             heavy_hitter_token_share=kw.get("heavy_share", 0.8),
                             inactive_expert_fraction=kw.get("inactive_fraction", 0.5))
    out = (C.c_uint32 * max(1, experts))()
    rc = cap.load().bmoe_generate_workload(C.byref(cfg), out)
    return rc, np.asarray(list(out)[:experts], dtype=np.uint32)


def test_generator_equals_golden_and_oracle(engine, oracle, golden):
    for name, entry in golden["workloads"].items():
        cfg = entry["config"]
        rc, counts = gen_counts(engine, cfg["experts"], cfg["total_tokens"], cfg["distribution"],
                                seed=cfg["seed"], zipf_alpha=cfg["zipf_alpha"],
                                heavy_fraction=cfg["heavy_fraction"], heavy_share=cfg["heavy_share"],
                                inactive_fraction=cfg["inactive_fraction"])
        assert rc == 0 and counts.tolist() == entry["counts"], name
    rng = np.random.default_rng(2)
    for _ in range(20):
        e, t, d = int(rng.integers(1, 200)), int(rng.integers(0, 20000)), int(rng.integers(0, 4))
        kw = dict(seed=int(rng.integers(0, 2**50)), zipf_alpha=float(rng.uniform(0.2, 2)))
        assert np.array_equal(gen_counts(engine, e, t, d, **kw)[1],
                              oracle.generate_counts(e, t, d, **kw)[1])
    # reference rejects these (src/workload/workload.cpp:64-76)
    assert gen_counts(engine, 0, 10, 0)[0] == engine._capi.INVALID_ARGUMENT
    assert gen_counts(engine, 8, 10, 3, zipf_alpha=0.0)[0] == engine._capi.INVALID_ARGUMENT
    assert gen_counts(engine, 8, 10, 1, heavy_fraction=0.0)[0] == engine._capi.INVALID_ARGUMENT
    assert gen_counts(engine, 8, 10, 2, inactive_fraction=1.5)[0] == engine._capi.INVALID_ARGUMENT


def test_heavy_sparse_family_equals_golden_and_oracle(engine, oracle, golden):
    """The decode-shaped routing family that exists only in this engine: hot set in front,
    idle set at the back. Golden counts come from the standard library's own generator
    objects over the stated weights."""
    for name, entry in golden["build_side_workloads"].items():
        cfg = entry["config"]
        kw = dict(seed=cfg["seed"], zipf_alpha=cfg["zipf_alpha"], heavy_fraction=cfg["heavy_fraction"],
                  heavy_share=cfg["heavy_share"], inactive_fraction=cfg["inactive_fraction"])
        rc, counts = gen_counts(engine, cfg["experts"], cfg["total_tokens"], 4, **kw)
        assert rc == 0 and counts.tolist() == entry["counts"], name
        rc, counts = oracle.generate_counts(cfg["experts"], cfg["total_tokens"], 4, **kw)
        assert rc == 0 and counts.tolist() == entry["counts"], name
        silent = int(np.floor(cfg["experts"] * cfg["inactive_fraction"]))
        assert not any(entry["counts"][cfg["experts"] - silent:])
    c3 = golden["build_side_workloads"]["c3_heavy_sparse_e256_decode"]
    assert sum(c3["counts"][:8]) / sum(c3["counts"]) == pytest.approx(0.5, abs=0.03)
    assert 150 <= c3["active_experts"] <= 154
    rng = np.random.default_rng(5)
    for _ in range(20):
        e, t = int(rng.integers(1, 300)), int(rng.integers(0, 20000))
        kw = dict(seed=int(rng.integers(0, 2**50)), heavy_fraction=float(rng.uniform(0.01, 1)),
                  heavy_share=float(rng.uniform(0, 1)), inactive_fraction=float(rng.uniform(0, 1)))
        assert np.array_equal(gen_counts(engine, e, t, 4, **kw)[1],
                              oracle.generate_counts(e, t, 4, **kw)[1]), (e, t, kw)
    assert gen_counts(engine, 8, 10, 5)[0] == engine._capi.INVALID_ARGUMENT


def test_workload_unit_expectations(engine):
    """tests/test_workload.cpp:18-57 of the reference."""
    for dist in range(4):
        rc, a = gen_counts(engine, 32, 10000, dist)
        rc2, b = gen_counts(engine, 32, 10000, dist)
        assert rc == rc2 == 0 and np.array_equal(a, b) and int(a.sum()) == 10000
    cap = engine._capi

    def metrics(counts, n=7168, tm=128, tn=128):
        out = cap.WorkloadMetrics()
        c = support.as_counts(counts)
        assert cap.load().bmoe_workload_metrics_compute(
            c.ctypes.data_as(C.POINTER(C.c_uint32)), len(c), n, tm, tn, C.byref(out)) == 0
        return out

    uni = metrics(gen_counts(engine, 32, 100000, 0)[1])
    heavy = metrics(gen_counts(engine, 32, 100000, 1)[1])
    assert heavy.coefficient_of_variation > uni.coefficient_of_variation
    exact = metrics([0, 64, 128, 256])
    assert abs(exact.inactive_expert_ratio - 0.25) < 1e-12
    assert abs(exact.small_m_expert_ratio - 0.25) < 1e-12


def test_metrics_equal_golden_bit_for_bit(engine, golden):
    cap = engine._capi
    for name, entry in golden["workloads"].items():
        n, tm, tn = entry["shape"]
        out = cap.WorkloadMetrics()
        c = support.as_counts(entry["counts"])
        cap.load().bmoe_workload_metrics_compute(c.ctypes.data_as(C.POINTER(C.c_uint32)), len(c),
                                                 n, tm, tn, C.byref(out))
        got = [out.mean_tokens, out.coefficient_of_variation, out.max_over_mean,
               out.inactive_expert_ratio, out.small_m_expert_ratio, out.tile_count_cv]
        assert [float(x).hex() for x in got] == entry["metrics"], name
        assert out.active_experts == entry["active_experts"]
        assert out.total_tiles == entry["total_tiles"]


def test_scheduler_unit_expectations(engine):
    """tests/test_scheduler.cpp:49-142 of the reference."""
    tokens = [0, 1, 128, 129]
    tiles = support.engine_host_tiles(engine, tokens, 256, 128, 128)
    assert len(tiles) == 8 and not np.any(tiles["expert_id"] == 0)
    tail = tiles[(tiles["expert_id"] == 3) & (tiles["tile_m"] == 1) & (tiles["tile_n"] == 0)]
    assert len(tail) == 1 and tail[0]["valid_m"] == 1 and tail[0]["valid_n"] == 128

    def same_tiles(a, b):
        return sorted(map(tuple, a.tolist())) == sorted(map(tuple, b.tolist()))

    for sched in (0, 1, 2):
        rc, flat, offs, _ = support.engine_simulate(engine, sched, tokens, 256, 128, 128, 3)
        assert rc == 0 and len(flat) == 8 and same_tiles(flat, tiles)
        if sched == 1:
            loads = np.diff(offs.astype(np.int64))
            assert loads.max() - loads.min() <= 1
    ordered = support.engine_host_tiles(engine, tokens, 256, 128, 128, order=1)
    assert ordered[0]["expert_id"] == 3

    rc, _, _, m = support.engine_simulate(engine, 0, [129], 129, 128, 128, 2)
    assert m.total_tiles == 4 and m.total_valid_elements == 129 * 129
    assert m.total_padded_elements == 4 * 128 * 128
    assert 0.25 < m.useful_work_ratio < 0.26 and m.tail_ratio > 1.0
    assert 0.0 < m.estimated_utilization <= 1.0

    _, _, _, m_static = support.engine_simulate(engine, 0, [1, 257, 129], 129, 128, 128, 3)
    _, _, _, m_dyn = support.engine_simulate(engine, 2, [1, 257, 129], 129, 128, 128, 3)
    assert m_dyn.tail_ratio < m_static.tail_ratio
    assert support.engine_simulate(engine, 2, tokens, 256, 128, 128, 0)[0] == engine._capi.INVALID_ARGUMENT
    assert support.engine_simulate(engine, 0, tokens, 256, 0, 128, 3)[0] == engine._capi.INVALID_ARGUMENT


def test_tiles_and_schedules_equal_golden(engine, golden):
    for case in golden["tile_cases"]:
        args = (case["counts"], case["n"], case["tile_m"], case["tile_n"])
        for order in (0, 1):
            tiles = support.engine_host_tiles(engine, *args, order=order)
            assert [list(map(int, t)) for t in tiles.tolist()] == case[f"order{order}"]
        for sched in range(5):
            want = case[f"sched{sched}_cta3"]
            rc, flat, offs, m = support.engine_simulate(engine, sched, *args, 3)
            assert rc == 0
            assert [list(map(int, t)) for t in flat.tolist()] == want["tiles"]
            assert [int(x) for x in offs] == want["offsets"]
            ints = [m.total_tiles, m.total_valid_elements, m.total_padded_elements,
                    m.expert_switches, m.min_tiles_per_cta, m.max_tiles_per_cta]
            reals = [m.mean_cta_work, m.max_cta_work, m.cta_work_cv, m.tail_ratio,
                     m.estimated_utilization, m.useful_work_ratio]
            assert ints == want["ints"]
            assert [float(x).hex() for x in reals] == want["reals"]
    for name, entry in golden["workloads"].items():
        n, tm, _ = entry["shape"]
        for tn in (128, 256):
            for order in (0, 1):
                tiles = support.engine_host_tiles(engine, entry["counts"], n, tm, tn, order=order)
                assert support.sha(tiles) == entry[f"tiles_sha256_tn{tn}_order{order}"]


def test_m_fastest_raster_is_a_per_expert_transpose(engine, oracle):
    rng = np.random.default_rng(5)
    for _ in range(10):
        e = int(rng.integers(1, 30))
        counts = (rng.integers(0, 700, size=e) * (rng.random(e) > 0.3)).astype(np.uint32)
        n = int(rng.integers(1, 1500))
        for order in (0, 1):
            ref = support.engine_host_tiles(engine, counts, n, 128, 256, order=order, raster=0)
            alt = support.engine_host_tiles(engine, counts, n, 128, 256, order=order, raster=1)
            assert np.array_equal(alt, oracle.build_tiles(counts, n, 128, 256, order=order, raster=1))
            assert sorted(map(tuple, ref.tolist())) == sorted(map(tuple, alt.tolist()))
            # same expert visiting order, tile_m fastest inside an expert
            assert [x for i, x in enumerate(ref["expert_id"]) if i == 0 or x != ref["expert_id"][i - 1]] == \
                   [x for i, x in enumerate(alt["expert_id"]) if i == 0 or x != alt["expert_id"][i - 1]]
            for ex in np.unique(alt["expert_id"]):
                sub = alt[alt["expert_id"] == ex]
                keys = list(zip(sub["tile_n"].tolist(), sub["tile_m"].tolist()))
                assert keys == sorted(keys)


def test_policy_names_round_trip(engine):
    names = engine._capi.SCHEDULER_NAMES
    assert names["sorted_static"] == names["static_persistent"] == 1
    assert names["clc"] == names["clc_assisted"] == 5 and names["baseline"] == 0


# ---- Python planner: expectations of the reference's tests/test_tirx_worklist.py ----

def test_planner_distributions_deterministic(engine):
    spec = engine.TIRxMoESpec(experts=16, tokens=1024, n=512, k=256)
    for dist in ("uniform", "heavy_hitter", "sparse", "zipf"):
        a = engine.build_workload_plan(spec, dist, seed=2026)
        b = engine.build_workload_plan(spec, dist, seed=2026)
        assert a.tokens_per_expert == b.tokens_per_expert and sum(a.tokens_per_expert) == 1024


def test_planner_compaction_and_order(engine):
    spec = engine.TIRxMoESpec(experts=4, tokens=290, n=256, k=64)
    plan = engine.build_workload_plan(spec, token_counts=(0, 1, 128, 161))
    assert plan.active_experts == 3 and plan.m_capacity == 256
    assert all(t.expert_id != 0 for t in plan.tiles)
    assert len(plan.tiles) == (1 + 1 + 2) * (spec.n // spec.tile_n)
    for ex, count in enumerate(plan.tokens_per_expert):
        rows = {t.tile_m: t.valid_m for t in plan.tiles if t.expert_id == ex and t.tile_n == 0}
        assert sum(rows.values()) == count
    spec2 = engine.TIRxMoESpec(experts=2, tokens=129, n=256, k=64)
    plan2 = engine.build_workload_plan(spec2, token_counts=(128, 1))
    assert plan2.device_worklist() == [[0, 0, 0], [0, 0, 1], [1, 0, 0], [1, 0, 1]]
    with pytest.raises(ValueError, match="128x128x64"):
        engine.TIRxMoESpec(tile_m=64).validate()
    with pytest.raises(ValueError):
        engine.build_workload_plan(spec2, token_counts=(128, 2))


def test_claim_models_equal_golden(engine, golden):
    flat = [t for cta in engine.static_cta_assignments(353, 148) for t in cta]
    assert sorted(flat) == list(range(353))
    assert support.sha(np.asarray(flat, dtype=np.int32)) == golden["planner"]["static_353_148_sha256"]
    for claim in (1, 2, 4, 8):
        got = [list(b) for b in engine.chunked_claims(353, claim)]
        assert got == golden["planner"]["chunked_353"][str(claim)]
    assert [list(b) for b in engine.hybrid_claims(353, 8, 37)] == golden["planner"]["hybrid_353_8_37"]
    with pytest.raises(ValueError):
        engine.chunked_claims(5, 0)


def test_registry_and_launch_contracts(engine, golden):
    assert list(engine.list_versions()) == golden["planner"]["versions"]
    want = golden["planner"]["launch_contracts"]
    spec = engine.TIRxMoESpec(experts=4, tokens=256, n=256, k=64, hybrid_tail_tiles=3)
    plan = engine.build_workload_plan(spec, token_counts=(64, 64, 64, 64))
    assert len(plan.tiles) == want["tiles"]
    for v in engine.list_versions():
        d = engine.get_descriptor(v)
        assert d.launch_ctas(spec, plan) == want["launch_ctas"][v]
        assert list(d.queue_initial_values(spec, plan)) == want["queue_init"][v]
        assert d.requires_queue == want["requires_queue"][v]
    with pytest.raises(ValueError):
        engine.get_descriptor("v9")


def test_dispatch_equals_reference_python(engine, golden):
    for case in golden["planner"]["feature_cases"]:
        spec = engine.TIRxMoESpec(**case["spec"])
        plan = engine.build_workload_plan(spec, token_counts=case["counts"])
        f = engine.routing_features(spec, plan)
        for key, want in case["features"].items():
            got = getattr(f, key)
            assert (float(got).hex() if isinstance(want, str) else int(got)) == want, (key, case["spec"])
        assert engine.select_kernel(spec, plan) == case["select_kernel"]
        assert plan.m_capacity == case["m_capacity"] and len(plan.tiles) == case["tile_count"]
        assert plan.logical_flops == case["logical_flops"]
        assert plan.padded_flops == case["padded_flops"]
        assert support.sha(np.asarray(plan.device_worklist(), dtype=np.int32)) == case["worklist_sha256"]


def test_harness_csv_schema_and_routing_files_match_the_reference(engine):
    """BenchmarkResult writes the reference harness's CSV (header and number formats
    pinned by a row the reference class formatted), and load_token_counts reads the
    files of the reference's generate_workloads.py."""
    import json
    from pathlib import Path

    golden_dir = Path(__file__).resolve().parent / "golden"
    golden = json.loads((golden_dir / "reference_vectors.json").read_text())["runner"]
    assert engine.BenchmarkResult.csv_header() == golden["csv_header"]
    assert engine.BenchmarkResult(**golden["sample_fields"]).csv_row() == golden["sample_row"]

    counts, name, seed = engine.load_token_counts(golden_dir / "workload_zipf_e16_t512.json")
    assert (len(counts), sum(counts), name, seed) == (16, 512, "zipf", 7)
    from_csv, csv_name, _ = engine.load_token_counts(golden_dir / "workload_zipf_e16_t512.csv")
    assert from_csv == counts and csv_name == "trace"
    spec = engine.MoESpec(experts=16, tokens=512, n=256, k=128)
    plan = engine.build_workload_plan(spec, name, seed=seed, token_counts=counts)
    assert plan.tokens_per_expert == counts and plan.distribution == "zipf"

    from bmoe_b200 import cli
    args = cli.build_parser().parse_args([])
    assert (args.kernel, args.experts, args.tokens, args.n, args.k, args.ctas, args.warmup,
            args.iterations) == ("v1_static_ws", 64, 4096, 7168, 2048, 148, 20, 200)
    with pytest.raises(ValueError):
        engine.run_benchmark(spec, plan, warmup=-1)


def test_fitted_dispatch_rule_on_the_benchmark_routings(engine, golden):
    """The rule a plan applies for `auto` (fitted on B200 measurements): launch control
    where tiles carry real rows, the static stride for weight-stream routings, one CTA per
    tile when no unit gets more than one. The reference's own rule keeps its answers."""
    cap = engine._capi
    lib = cap.load()

    def pick(counts, n, tile_m, tile_n, units, rule=None):
        c = support.as_counts(counts)
        f = cap.RoutingFeatures()
        assert lib.bmoe_routing_features_compute(c.ctypes.data_as(C.POINTER(C.c_uint32)), len(c), n,
                                                 tile_m, tile_n, units, C.byref(f)) == 0
        out = C.c_uint32(99)
        arr = (C.c_double * 2)(*rule) if rule else None
        assert lib.bmoe_select_variant_fitted(C.byref(f), arr, C.byref(out)) == 0
        return cap.VARIANT_NAMES[out.value]

    w = golden["workloads"]
    assert pick(w["c2_zipf1_e8"]["counts"], 14336, 256, 256, 74) == "v5_clc"
    for name in ("c4_uniform_e128", "c4_zipf05_e128", "c4_zipf10_e128", "c4_zipf15_e128"):
        assert pick(w[name]["counts"], 768, 256, 256, 74) == "v5_clc", name
    assert pick(w["zipf_e64_default"]["counts"], 7168, 128, 256, 148) == "v5_clc"
    decode = golden["build_side_workloads"]["c3_heavy_sparse_e256_decode"]["counts"]
    assert pick(decode, 2048, 128, 256, 148) == "v1_static_ws"       # 13 rows per active expert
    assert pick(w["c1_uniform_e8"]["counts"], 1024, 128, 128, 148) == "v0_nonpersistent"
    assert pick(decode, 2048, 128, 256, 148, rule=(1.0, 4.0)) == "v5_clc"
    assert lib.bmoe_select_variant_fitted(None, None, None) == cap.INVALID_ARGUMENT
