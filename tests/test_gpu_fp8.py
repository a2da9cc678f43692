"""FP8 E4M3 grouped GEMM on the GPU through the C interface, against the CPU oracle.

The reference declares the type (include/blackwell_moe/kernels/grouped_gemm.cuh:10) and
rejects it in every implementation (baselines/cutlass/cutlass_baseline.cu:211-213), so no
reference result exists to compare with. The contract tested here is the engine's: both
operands one byte per element, decoded exactly, no scales, FP32 accumulation, BF16 (or
FP32) output. The oracle decodes the bytes to BF16 bit patterns (exact) and runs the BF16
contract's FP32 sequential-k loop. Bars as for BF16: every launch variant bit-identical
to expert order; max |err| <= 2 BF16 ulp of the unrounded FP32 reference (ulp taken at
max(|ref|, 2^-6)); relative Frobenius error <= 1e-3 against the oracle's BF16 output."""

import numpy as np
import pytest

import support
from test_gpu_gemm import POLICIES, bits_of

pytestmark = pytest.mark.gpu


def make_fp8_inputs(counts, n, k, seed=2026, device="cpu"):
    """A ~ N(0,1), W ~ N(0,1) / sqrt(k) * 8 rounded to E4M3 by torch (the factor 8 keeps the
    weights out of the subnormal range for the larger k); returned as uint8 bit patterns."""
    import torch

    gen = torch.Generator(device=device).manual_seed(seed)
    rows = sum(counts)
    a = torch.randn(max(1, rows), k, generator=gen, device=device)[:rows]
    a = a.to(torch.float8_e4m3fn).view(torch.uint8)
    w = torch.empty(len(counts), n, k, dtype=torch.uint8, device=device)
    for e in range(len(counts)):
        w[e] = (torch.randn(n, k, generator=gen, device=device) * (8.0 * k ** -0.5)).to(
            torch.float8_e4m3fn).view(torch.uint8)
    return a, w


def run_fp8(engine, a, w, counts, policy="expert_order", *, output_f32=False, **options):
    import torch

    n = w.shape[1]
    a_dev, w_dev = a.cuda(), w.cuda()
    d_dev = torch.full((max(1, sum(counts)), n), float("nan"),
                       dtype=torch.float32 if output_f32 else torch.bfloat16,
                       device="cuda")[: sum(counts)]
    visits = None
    plan = engine.GroupedGemmPlan()
    try:
        status = plan.initialize_packed(a_dev, w_dev, d_dev, counts, scheduler=policy,
                                        output_f32=output_f32, **options)
        assert status == 0, engine._capi.status_string(status)
        stats = plan.stats()
        if stats.total_tiles:
            visits = torch.zeros(stats.total_tiles, dtype=torch.int32, device="cuda")
            assert plan.set_observers(visits, None) == 0
        assert plan.run() == 0
        status, report = plan.poll()
        assert status == 0, (engine._capi.status_string(status), report.code, report.cta,
                             report.role, report.tile, report.stage, report.aux)
        out = d_dev.cpu().numpy() if output_f32 else bits_of(d_dev)
        return {"out": out, "stats": stats,
                "visits": None if visits is None else visits.cpu().numpy()}
    finally:
        plan.close()


def check_fp8_against_oracle(oracle, a, w, counts, got_bits, rows=None, row_stride=1,
                             row_phase=0):
    n, k = w.shape[1], w.shape[2]
    a_bits = oracle.e4m3_to_bf16(a.cpu().numpy())
    w_bits = oracle.e4m3_to_bf16(w.cpu().numpy())
    ref = oracle.grouped_gemm(a_bits, w_bits, counts, n, k, want_f32=True,
                              row_stride=row_stride, row_phase=row_phase)
    pick = slice(None) if rows is None else rows
    exact = ref["f32"][pick].astype(np.float64)
    got = support.bf16_bits_to_f32(got_bits[pick]).astype(np.float64)
    assert np.all(np.isfinite(support.bf16_bits_to_f32(got_bits))), "unwritten outputs"
    mag = np.maximum(np.abs(exact), 2.0 ** -6)
    err_ulp = (np.abs(got - exact) / 2.0 ** (np.floor(np.log2(mag)) - 7)).max()
    assert err_ulp <= 2.0, f"max error {err_ulp:.3f} BF16 ulp"
    want = support.bf16_bits_to_f32(ref["bf16"][pick]).astype(np.float64)
    rel_fro = np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-30)
    assert rel_fro <= 1e-3, f"relative Frobenius error {rel_fro:.3e}"
    return ref


FP8_CASES = [
    # counts, n, k (k a multiple of 16: a row of k bytes is a tensor-map stride)
    ([1], 8, 16),
    ([128], 256, 128),
    ([129, 0, 1, 255], 264, 80),
    ([37, 0, 1, 200], 384, 192),
    ([300, 5, 0, 300, 129], 520, 448),
    ([65, 67, 68, 61, 63, 57, 61, 70], 1024, 512),
    ([3] * 40 + [0] * 20 + [500], 256, 1024),
]


@pytest.mark.parametrize("counts,n,k", FP8_CASES)
def test_fp8_ragged_cases_all_variants(engine, oracle, counts, n, k):
    """Ragged experts, ragged n and k (k not a multiple of the 128-byte k-block), every
    tile shape, CTA group, raster and policy: one result, equal to the oracle's."""
    a, w = make_fp8_inputs(counts, n, k)
    base = run_fp8(engine, a, w, counts, "expert_order", raster_along_m=0)
    check_fp8_against_oracle(oracle, a, w, counts, base["out"])
    assert np.all(base["visits"] == 1)
    for tile_n, group in ((64, 1), (128, 1), (256, 1), (256, 2)):
        for raster in (0, 1):
            for policy, opts in POLICIES:
                out = run_fp8(engine, a, w, counts, policy, tile_n=tile_n, cta_group=group,
                              raster_along_m=raster, **opts)
                key = (policy, opts, tile_n, group, raster)
                assert np.array_equal(out["out"], base["out"]), key
                assert np.all(out["visits"] == 1), key


def test_fp8_products_are_summed_in_fp32(engine, oracle):
    """The FP32 epilogue shows the accumulators themselves: against the FP64 sum of the
    exact products the error stays within FP32 accumulation of k terms (1e-5 of the
    row's sum of |products|), for single CTAs and CTA pairs, which agree bit for bit."""
    counts, n, k = [200, 0, 77], 512, 1024
    a, w = make_fp8_inputs(counts, n, k, seed=7)
    single = run_fp8(engine, a, w, counts, output_f32=True, cta_group=1, tile_n=256)
    pair = run_fp8(engine, a, w, counts, output_f32=True, cta_group=2, tile_n=256)
    assert np.array_equal(single["out"].view(np.uint32), pair["out"].view(np.uint32))
    a_f = support.bf16_bits_to_f32(oracle.e4m3_to_bf16(a.numpy())).astype(np.float64)
    w_f = support.bf16_bits_to_f32(oracle.e4m3_to_bf16(w.numpy())).astype(np.float64)
    row0 = 0
    for e, m in enumerate(counts):
        if m == 0:
            continue
        exact = a_f[row0:row0 + m] @ w_f[e].T
        scale = np.abs(a_f[row0:row0 + m]) @ np.abs(w_f[e]).T
        err = np.abs(single["out"][row0:row0 + m].astype(np.float64) - exact)
        assert (err / scale).max() <= 1e-5, (e, float((err / scale).max()))
        row0 += m


def test_fp8_equals_bf16_engine_on_the_decoded_operands(engine, oracle):
    """Decoding E4M3 to BF16 is exact, so the BF16 engine on the decoded operands computes
    the same sums of the same products; both results lie within the bars of the same
    oracle output, and they differ from each other by at most one BF16 rounding step."""
    import torch

    from test_gpu_gemm import run_engine

    counts, n, k = [300, 5, 0, 300, 129], 520, 448
    a, w = make_fp8_inputs(counts, n, k, seed=11)
    fp8 = run_fp8(engine, a, w, counts)["out"]
    a16 = torch.from_numpy(oracle.e4m3_to_bf16(a.numpy()).view(np.int16)).view(torch.bfloat16)
    w16 = torch.from_numpy(oracle.e4m3_to_bf16(w.numpy()).view(np.int16)).view(torch.bfloat16)
    bf16 = run_engine(engine, a16, w16, counts)["bits"]
    check_fp8_against_oracle(oracle, a, w, counts, fp8)
    check_fp8_against_oracle(oracle, a, w, counts, bf16)
    x = support.bf16_bits_to_f32(fp8).astype(np.float64)
    y = support.bf16_bits_to_f32(bf16).astype(np.float64)
    mag = np.maximum(np.maximum(np.abs(x), np.abs(y)), 2.0 ** -6)
    assert (np.abs(x - y) / 2.0 ** (np.floor(np.log2(mag)) - 7)).max() <= 1.0


def test_fp8_benchmark_shape_properties(engine, oracle, golden):
    """The Mixtral-shaped headline routing at full size with FP8 operands (E=8, 8192 routed
    rows, K=4096, N=14336): variants bit-identical, every tile once, a row sample within
    the bars of the oracle."""
    counts, n, k = golden["workloads"]["c2_zipf1_e8"]["counts"], 14336, 4096
    a, w = make_fp8_inputs(counts, n, k, device="cuda")
    base = run_fp8(engine, a, w, counts, "expert_order")
    assert np.all(base["visits"] == 1)
    for policy, opts in [("static_persistent", {}), ("dynamic_queue", {"claim_size": 4}),
                         ("clc", {}), ("auto", {}), ("expert_order", {"cta_group": 1}),
                         ("dynamic_queue", {"cta_group": 2}), ("clc", {"cta_group": 2})]:
        out = run_fp8(engine, a, w, counts, policy, **opts)
        assert np.array_equal(out["out"], base["out"]), (policy, opts)
        assert np.all(out["visits"] == 1), (policy, opts)
    stride, phase = 257, 3
    rows, row0 = [], 0
    for m in counts:
        rows.extend(range(row0 + phase, row0 + m, stride))
        row0 += m
    check_fp8_against_oracle(oracle, a, w, counts, base["out"], rows=rows, row_stride=stride,
                             row_phase=phase)


def test_fp8_argument_rules(engine):
    """k must be a multiple of 16 (tensor-map stride); unknown type codes are refused."""
    import torch

    cap = engine._capi
    a = torch.zeros(8, 40, dtype=torch.uint8, device="cuda")
    w = torch.zeros(1, 8, 40, dtype=torch.uint8, device="cuda")
    d = torch.zeros(8, 8, dtype=torch.bfloat16, device="cuda")
    plan = engine.GroupedGemmPlan()
    try:
        assert plan.initialize_packed(a, w, d, [8]) == cap.INVALID_ARGUMENT
        assert plan.initialize([a.data_ptr()], [w.data_ptr()], [d.data_ptr()], [8], 8, 48,
                               data_type=2) == cap.UNSUPPORTED_DATA_TYPE
    finally:
        plan.close()
