"""Generates tests/golden/reference_vectors.json from the REFERENCE itself.

Run where the reference checkout is present (its location: BMOE_REFERENCE_ROOT):
    python tests/golden/make_golden.py
Sources of truth:
  * the reference's compiled host scheduler (oracle/_ref/libref_sched.so, built
    by oracle/build_oracle.py from the reference's own .cpp files)
  * the reference's pure-Python planner (python/blackwell_moe_tirx/config.py,
    dispatch.py, kernels/registry.py), imported from the checkout
  * the reference's GEMM known-answer inputs (formulas in
    baselines/cutlass/test_correctness.cu:73-80 and
    tests/test_sm100_*_correctness.cu), whose products are multiples of 1/256
    with |sum| small enough to be exact in FP32; the expected BF16 output is
    therefore fixed by arithmetic and is computed here in float64.
  * "build_side_workloads": routing families that exist only in this engine (the
    heavy_sparse family of the decode-shaped configuration). Their weights are
    stated here and drawn through the reference's draw loop over the same
    standard-library generator objects (ref_draw_counts in oracle/ref_shim.cpp).
The JSON is committed; tests never read the reference checkout.
"""

from __future__ import annotations

import ctypes
import hashlib
import json
import os
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
REFERENCE = Path(os.environ.get("BMOE_REFERENCE_ROOT", "/root/reference"))

sys.path.insert(0, str(ROOT / "oracle"))
import build_oracle  # noqa: E402

TILE_DTYPE = np.dtype([("expert_id", "<u4"), ("tile_m", "<u4"), ("tile_n", "<u4"),
                       ("valid_m", "<u4"), ("valid_n", "<u4")])


def sha(arr: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(arr).tobytes()).hexdigest()


def main() -> None:
    ref_path = build_oracle.build_reference()
    assert ref_path is not None and build_oracle.reference_available()
    ref = ctypes.CDLL(str(ref_path))
    ref.ref_build_tiles.restype = ctypes.c_uint64
    ref.ref_simulate.restype = ctypes.c_uint64
    u32, u64, f64 = ctypes.c_uint32, ctypes.c_uint64, ctypes.c_double

    def counts_for(cfg):
        out = np.zeros(cfg["experts"], dtype=np.uint32)
        rc = ref.ref_generate_counts(
            u32(cfg["experts"]), u64(cfg["total_tokens"]), u32(cfg["distribution"]),
            u64(cfg["seed"]), f64(cfg["zipf_alpha"]), f64(cfg["heavy_fraction"]),
            f64(cfg["heavy_share"]), f64(cfg["inactive_fraction"]),
            out.ctypes.data_as(ctypes.c_void_p))
        assert rc == 0
        return out

    def tiles_for(counts, n, tm, tn, order):
        total = ref.ref_build_tiles(counts.ctypes.data_as(ctypes.c_void_p), u32(len(counts)),
                                    u32(n), u32(tm), u32(tn), u32(order), None, u64(0))
        buf = np.zeros(max(1, total), dtype=TILE_DTYPE)
        ref.ref_build_tiles(counts.ctypes.data_as(ctypes.c_void_p), u32(len(counts)),
                            u32(n), u32(tm), u32(tn), u32(order),
                            buf.ctypes.data_as(ctypes.c_void_p), u64(total))
        return buf[:total]

    def simulate(sched, counts, n, tm, tn, ctas):
        total = len(tiles_for(counts, n, tm, tn, 0))
        buf = np.zeros(max(1, total), dtype=TILE_DTYPE)
        offs = np.zeros(ctas + 1, dtype=np.uint64)
        ints = np.zeros(6, dtype=np.uint64)
        reals = np.zeros(6, dtype=np.float64)
        got = ref.ref_simulate(u32(sched), counts.ctypes.data_as(ctypes.c_void_p),
                               u32(len(counts)), u32(n), u32(tm), u32(tn), u32(ctas),
                               buf.ctypes.data_as(ctypes.c_void_p), u64(total),
                               offs.ctypes.data_as(ctypes.c_void_p),
                               ints.ctypes.data_as(ctypes.c_void_p),
                               reals.ctypes.data_as(ctypes.c_void_p))
        assert got == total
        return buf[:total], offs, ints, reals

    def metrics(counts, n, tm, tn):
        out = np.zeros(6, dtype=np.float64)
        oi = np.zeros(2, dtype=np.uint64)
        ref.ref_workload_metrics(counts.ctypes.data_as(ctypes.c_void_p), u32(len(counts)),
                                 u32(n), u32(tm), u32(tn),
                                 out.ctypes.data_as(ctypes.c_void_p),
                                 oi.ctypes.data_as(ctypes.c_void_p))
        return out, oi

    base = dict(seed=2026, zipf_alpha=1.2, heavy_fraction=0.1, heavy_share=0.8,
                inactive_fraction=0.5)
    # Workloads of the benchmark configurations plus the reference test cases.
    workload_cfgs = {
        "c1_uniform_e8": dict(base, experts=8, total_tokens=512, distribution=0),
        "c2_zipf1_e8": dict(base, experts=8, total_tokens=8192, distribution=3, zipf_alpha=1.0),
        "c4_zipf05_e128": dict(base, experts=128, total_tokens=131072, distribution=3, zipf_alpha=0.5),
        "c4_zipf10_e128": dict(base, experts=128, total_tokens=131072, distribution=3, zipf_alpha=1.0),
        "c4_zipf15_e128": dict(base, experts=128, total_tokens=131072, distribution=3, zipf_alpha=1.5),
        "c4_uniform_e128": dict(base, experts=128, total_tokens=131072, distribution=0),
        "c5_zipf1_e256": dict(base, experts=256, total_tokens=262144, distribution=3, zipf_alpha=1.0),
        "heavy_e32": dict(base, experts=32, total_tokens=10000, distribution=1),
        "sparse_e32": dict(base, experts=32, total_tokens=10000, distribution=2),
        "zipf_e64_default": dict(base, experts=64, total_tokens=4096, distribution=3),
        "heavy_e256_decode": dict(base, experts=256, total_tokens=2048, distribution=1,
                                  heavy_fraction=8 / 256, heavy_share=0.5),
    }
    shapes = {
        "c1_uniform_e8": (1024, 128, 128), "c2_zipf1_e8": (14336, 128, 128),
        "c4_zipf05_e128": (768, 128, 128), "c4_zipf10_e128": (768, 128, 128),
        "c4_zipf15_e128": (768, 128, 128), "c4_uniform_e128": (768, 128, 128),
        "c5_zipf1_e256": (2048, 128, 128), "heavy_e32": (7168, 128, 128),
        "sparse_e32": (7168, 128, 128), "zipf_e64_default": (7168, 128, 128),
        "heavy_e256_decode": (2048, 128, 128),
    }
    out = {"workloads": {}, "tile_cases": [], "schedules": [], "planner": {}, "gemm_kats": {}}
    for name, cfg in workload_cfgs.items():
        counts = counts_for(cfg)
        n, tm, tn = shapes[name]
        m, mi = metrics(counts, n, tm, tn)
        entry = {"config": cfg, "shape": [n, tm, tn], "counts": counts.tolist(),
                 "metrics": [float(x).hex() for x in m],
                 "active_experts": int(mi[0]), "total_tiles": int(mi[1])}
        for tn2 in (128, 256):
            for order in (0, 1):
                t = tiles_for(counts, n, tm, tn2, order)
                entry[f"tiles_sha256_tn{tn2}_order{order}"] = sha(t)
                entry[f"tiles_count_tn{tn2}"] = int(len(t))
        sched = {}
        for s in (0, 1, 2):
            if s == 2 and len(tiles_for(counts, n, tm, tn, 0)) > 8000:
                continue  # the O(tiles x CTAs) ideal queue is checked on the smaller cases
            tiles, offs, ints, reals = simulate(s, counts, n, tm, tn, 148)
            sched[str(s)] = {"tiles_sha256": sha(tiles), "offsets_sha256": sha(offs),
                             "ints": [int(x) for x in ints],
                             "reals": [float(x).hex() for x in reals]}
        entry["schedule_148"] = sched
        out["workloads"][name] = entry

    # ---- engine-side routing families (no generator in the reference) ----
    # heavy_sparse: the first ceil(E * heavy_fraction) experts share heavy_share, the
    # last floor(E * inactive_fraction) experts get nothing, the rest share evenly.
    out["build_side_workloads"] = {}
    for name, cfg, shape in [
        ("c3_heavy_sparse_e256_decode",
         dict(base, experts=256, total_tokens=2048, distribution=4, heavy_fraction=8 / 256,
              heavy_share=0.5, inactive_fraction=0.4), (2048, 128, 128)),
        ("heavy_sparse_e32", dict(base, experts=32, total_tokens=10000, distribution=4),
         (7168, 128, 128)),
    ]:
        e = cfg["experts"]
        silent = min(e - 1, int(np.floor(e * cfg["inactive_fraction"])))
        heavy = min(e - silent, max(1, int(np.ceil(e * cfg["heavy_fraction"]))))
        light = e - silent - heavy
        weights = np.zeros(e, dtype=np.float64)
        weights[:heavy] = (cfg["heavy_share"] if light else 1.0) / heavy
        if light:
            weights[heavy:heavy + light] = (1.0 - cfg["heavy_share"]) / light
        counts = np.zeros(e, dtype=np.uint32)
        rc = ref.ref_draw_counts(weights.ctypes.data_as(ctypes.c_void_p), u32(e),
                                 u64(cfg["total_tokens"]), u64(cfg["seed"]),
                                 counts.ctypes.data_as(ctypes.c_void_p))
        assert rc == 0 and int(counts.sum()) == cfg["total_tokens"]
        n, tm, tn = shape
        m, mi = metrics(counts, n, tm, tn)
        entry = {"config": cfg, "shape": [n, tm, tn], "counts": counts.tolist(),
                 "metrics": [float(x).hex() for x in m],
                 "active_experts": int(mi[0]), "total_tiles": int(mi[1])}
        for tn2 in (128, 256):
            for order in (0, 1):
                entry[f"tiles_sha256_tn{tn2}_order{order}"] = sha(tiles_for(counts, n, tm, tn2, order))
        out["build_side_workloads"][name] = entry

    # Small explicit tile cases (full records), incl. the reference's unit-test inputs.
    for counts, n, tm, tn in [([0, 1, 128, 129], 256, 128, 128), ([129], 129, 128, 128),
                              ([1, 257, 129], 129, 128, 128), ([7, 0, 13, 31], 32, 128, 128),
                              ([0, 0, 0], 256, 128, 128), ([300, 5, 0, 300, 129], 520, 128, 256),
                              ([5, 5, 5, 5], 128, 128, 128), ([128, 1], 256, 128, 128),
                              ([1000, 3, 64, 1000, 2, 999], 384, 64, 96)]:
        c = np.asarray(counts, dtype=np.uint32)
        case = {"counts": counts, "n": n, "tile_m": tm, "tile_n": tn}
        for order in (0, 1):
            t = tiles_for(c, n, tm, tn, order)
            case[f"order{order}"] = [[int(x) for x in rec] for rec in t.tolist()]
        for s in (0, 1, 2, 3, 4):
            tiles, offs, ints, reals = simulate(s, c, n, tm, tn, 3)
            case[f"sched{s}_cta3"] = {
                "tiles": [[int(x) for x in rec] for rec in tiles.tolist()],
                "offsets": [int(x) for x in offs], "ints": [int(x) for x in ints],
                "reals": [float(x).hex() for x in reals]}
        out["tile_cases"].append(case)

    # ---- reference Python planner / dispatch ----
    sys.path.insert(0, str(REFERENCE / "python"))
    from blackwell_moe_tirx.config import (TIRxMoESpec, build_workload_plan, chunked_claims,
                                           hybrid_claims, static_cta_assignments)
    from blackwell_moe_tirx.dispatch import routing_features, select_kernel
    from blackwell_moe_tirx.kernels import get_descriptor, list_versions

    feature_cases = []
    rng = np.random.default_rng(7)
    specs = [
        (dict(experts=4, tokens=256, n=256, k=64, cta_count=2), (64, 64, 64, 64)),
        (dict(experts=4, tokens=4, n=128, k=64, cta_count=148), (1, 1, 1, 1)),
        (dict(experts=4, tokens=290, n=256, k=64), (0, 1, 128, 161)),
        (dict(experts=8, tokens=8192, n=14336, k=4096),
         tuple(out["workloads"]["c2_zipf1_e8"]["counts"])),
        (dict(experts=128, tokens=131072, n=768, k=2048),
         tuple(out["workloads"]["c4_zipf15_e128"]["counts"])),
        (dict(experts=128, tokens=131072, n=768, k=2048),
         tuple(out["workloads"]["c4_uniform_e128"]["counts"])),
        (dict(experts=256, tokens=2048, n=2048, k=7168),
         tuple(out["workloads"]["heavy_e256_decode"]["counts"])),
        (dict(experts=32, tokens=10000, n=7168, k=2048),
         tuple(out["workloads"]["sparse_e32"]["counts"])),
    ]
    for _ in range(24):
        e = int(rng.integers(1, 40))
        counts = tuple(int(x) for x in rng.integers(0, 700, size=e) * (rng.random(e) > 0.3))
        specs.append((dict(experts=e, tokens=sum(counts), n=int(rng.integers(1, 12)) * 128,
                           k=64 * int(rng.integers(1, 8)),
                           cta_count=int(rng.integers(1, 200))), counts))
    for kw, counts in specs:
        spec = TIRxMoESpec(**kw)
        plan = build_workload_plan(spec, token_counts=counts)
        f = routing_features(spec, plan)
        feature_cases.append({
            "spec": kw, "counts": list(counts),
            "features": {k: (float(v).hex() if isinstance(v, float) else int(v))
                         for k, v in f.__dict__.items()},
            "select_kernel": select_kernel(spec, plan),
            "m_capacity": plan.m_capacity, "tile_count": len(plan.tiles),
            "logical_flops": plan.logical_flops, "padded_flops": plan.padded_flops,
            "worklist_sha256": sha(np.asarray(plan.device_worklist(), dtype=np.int32)),
        })
    out["planner"]["feature_cases"] = feature_cases
    out["planner"]["versions"] = list(list_versions())
    out["planner"]["static_353_148_sha256"] = sha(np.asarray(
        [t for cta in static_cta_assignments(353, 148) for t in cta], dtype=np.int32))
    out["planner"]["chunked_353"] = {str(c): [list(b) for b in chunked_claims(353, c)]
                                     for c in (1, 2, 4, 8)}
    out["planner"]["hybrid_353_8_37"] = [list(b) for b in hybrid_claims(353, 8, 37)]
    hs = TIRxMoESpec(experts=4, tokens=256, n=256, k=64, hybrid_tail_tiles=3)
    hp = build_workload_plan(hs, token_counts=(64, 64, 64, 64))
    out["planner"]["launch_contracts"] = {
        "tiles": len(hp.tiles),
        "launch_ctas": {v: get_descriptor(v).launch_ctas(hs, hp) for v in list_versions()},
        "queue_init": {v: list(get_descriptor(v).queue_initial_values(hs, hp))
                       for v in list_versions()},
        "requires_queue": {v: get_descriptor(v).requires_queue for v in list_versions()},
    }

    # ---- GEMM known-answer cases: inputs by formula, outputs exact ----
    def bf16_bits(x64: np.ndarray) -> np.ndarray:
        f = x64.astype(np.float32)
        u = f.view(np.uint32)
        r = u + 0x7FFF + ((u >> 16) & 1)
        return (r >> 16).astype(np.uint16)

    def kat(name, counts, n, k, fa, fb, div):
        d_all = []
        for e, m in enumerate(counts):
            if m == 0:
                continue
            ia = np.arange(m * k, dtype=np.int64)
            ib = np.arange(n * k, dtype=np.int64)
            a = (fa(ia, e) / div).reshape(m, k)
            b = (fb(ib, e) / div).reshape(n, k)
            d_all.append(bf16_bits(a @ b.T).reshape(-1))
        bits = np.concatenate(d_all)
        out["gemm_kats"][name] = {"counts": counts, "n": n, "k": k,
                                  "d_sha256": sha(bits), "d_first16": bits[:16].tolist(),
                                  "d_elems": int(bits.size)}

    kat("cutlass_baseline_kat", [7, 0, 13, 31], 32, 32,
        lambda i, e: ((i + 3 * e) % 11 - 5).astype(np.float64),
        lambda i, e: ((3 * i + e) % 13 - 6).astype(np.float64), 8.0)
    kat("sm100_dense_kat", [128], 128, 64,
        lambda i, e: (i % 9 - 4).astype(np.float64),
        lambda i, e: ((3 * i) % 11 - 5).astype(np.float64), 16.0)
    kat("sm100_2sm_kat", [256], 128, 64,
        lambda i, e: (i % 7 - 3).astype(np.float64),
        lambda i, e: ((5 * i) % 13 - 6).astype(np.float64), 16.0)

    # ---- data formats of the reference's Python harness ----
    # CSV schema of blackwell_moe_tirx/runner.py (header and the formatting of one
    # row built from fixed field values), and one routing file written by
    # python/generate_workloads.py (JSON and CSV form) for the ingestion test.
    from blackwell_moe_tirx.runner import BenchmarkResult
    sample = dict(
        device="NVIDIA B200", implementation="impl_name", acquisition="global atomic queue; claim 1",
        distribution="zipf", experts=64, active_experts=61, tokens=4096, n=7168, k=2048,
        tiles=3584, ctas=148, pipe_depth=2, claim_size=4, hybrid_main_claim_size=8,
        hybrid_tail_tiles=296, cv_m=1.23456789, max_over_mean_m=7.5, inactive_expert_ratio=0.046875,
        small_m_expert_ratio=0.75, expert_tile_cv=1.1, max_expert_tiles_over_mean=6.25,
        tiles_per_cta=24.2162162, useful_work_ratio=0.8765432, median_ms=0.32691, p95_ms=0.3400004,
        effective_tflops=367.94449, max_abs_error=0.0078125, max_rel_error=1.25e-05)
    out["runner"] = {"csv_header": BenchmarkResult.csv_header(),
                     "sample_fields": sample,
                     "sample_row": BenchmarkResult(**sample).csv_row()}
    import subprocess
    script = REFERENCE / "python" / "generate_workloads.py"
    flags = ["--distribution", "zipf", "--experts", "16", "--tokens", "512", "--seed", "7",
             "--zipf-alpha", "1.1"]
    for fmt in ("json", "csv"):
        text = subprocess.run([sys.executable, str(script), *flags, "--format", fmt],
                              check=True, capture_output=True, text=True).stdout
        (HERE / f"workload_zipf_e16_t512.{fmt}").write_text(text)

    path = HERE / "reference_vectors.json"
    path.write_text(json.dumps(out, indent=1, sort_keys=True) + "\n")
    print(f"wrote {path} ({path.stat().st_size} bytes)")


if __name__ == "__main__":
    main()
