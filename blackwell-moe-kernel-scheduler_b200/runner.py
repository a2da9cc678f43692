"""Correctness and CUDA-event benchmark harness of the grouped-GEMM engine.

Host-side mirror of the reference's Python harness
(python/blackwell_moe_tirx/runner.py:15-88 ``BenchmarkResult`` with its CSV
schema, :234-339 ``run_benchmark``): same call, same result record, same CSV
header and number formatting, so a result file of either harness loads with the
other's tooling. Where the reference compiles one TIRx kernel per workload, this
harness initialises one plan of the precompiled sm_100a kernel in the launch
variant the version name stands for.

Differences that the record states itself: ``implementation`` names the engine's
variant, ``ctas`` and ``pipe_depth`` are what the engine actually launched
(CTAs of the grid, operand stages in shared memory).
"""

from __future__ import annotations

import json
import math
import statistics
from dataclasses import dataclass, fields
from pathlib import Path
from typing import Sequence

from .planner import MoESpec, MoEWorkloadPlan, get_descriptor, routing_features


@dataclass(frozen=True)
class BenchmarkResult:
    device: str
    implementation: str
    acquisition: str
    distribution: str
    experts: int
    active_experts: int
    tokens: int
    n: int
    k: int
    tiles: int
    ctas: int
    pipe_depth: int
    claim_size: int
    hybrid_main_claim_size: int
    hybrid_tail_tiles: int
    cv_m: float
    max_over_mean_m: float
    inactive_expert_ratio: float
    small_m_expert_ratio: float
    expert_tile_cv: float
    max_expert_tiles_over_mean: float
    tiles_per_cta: float
    useful_work_ratio: float
    median_ms: float
    p95_ms: float
    effective_tflops: float
    max_abs_error: float
    max_rel_error: float

    # Column formats of the reference's CSV (runner.py:57-88): plain for strings and
    # integers, six decimals for ratios and milliseconds, three for TFLOP/s, six
    # significant digits for the errors.
    _FORMATS = {"effective_tflops": "{:.3f}", "max_abs_error": "{:.6g}", "max_rel_error": "{:.6g}"}

    @classmethod
    def csv_header(cls) -> str:
        return ",".join(f.name for f in fields(cls))

    def csv_row(self) -> str:
        cells = []
        for f in fields(self):
            value = getattr(self, f.name)
            if isinstance(value, float):
                cells.append(self._FORMATS.get(f.name, "{:.6f}").format(value))
            else:
                cells.append(str(value))
        return ",".join(cells)


def load_token_counts(path) -> tuple[tuple[int, ...], str, int]:
    """Routing file written by the reference's ``python/generate_workloads.py`` (:54-58):
    JSON ``{"distribution", "seed", "tokens_per_expert"}`` or CSV ``expert_id,tokens``.
    Returns (counts, distribution, seed); the CSV form carries neither name nor seed."""
    path = Path(path)
    text = path.read_text(encoding="utf-8")
    if text.lstrip().startswith("{"):
        doc = json.loads(text)
        counts = tuple(int(c) for c in doc["tokens_per_expert"])
        return counts, str(doc.get("distribution", "trace")), int(doc.get("seed", 0))
    lines = [ln.strip() for ln in text.splitlines() if ln.strip()]
    if not lines or lines[0].replace(" ", "") != "expert_id,tokens":
        raise ValueError(f"{path}: expected JSON or a CSV with the header expert_id,tokens")
    pairs = [tuple(int(x) for x in ln.split(",")) for ln in lines[1:]]
    if [e for e, _ in pairs] != list(range(len(pairs))):
        raise ValueError(f"{path}: expert ids must be 0..E-1 in order")
    return tuple(t for _, t in pairs), "trace", 0


def percentile_95(values: Sequence[float]) -> float:
    """``sorted[ceil(0.95 n) - 1]`` as in the reference (runner.py:129-133)."""
    if not values:
        return math.nan
    ordered = sorted(values)
    return ordered[math.ceil(0.95 * len(ordered)) - 1]


def run_benchmark(
    spec: MoESpec,
    plan: MoEWorkloadPlan,
    *,
    version: str = "v1_static_ws",
    warmup: int = 20,
    iterations: int = 200,
    correctness_only: bool = False,
    dump_cuda: Path | None = None,
    **plan_options,
) -> BenchmarkResult:
    """Initialise once, enforce correctness, then report median and p95 latency of
    ``run()`` alone (CUDA events per launch, as runner.py:276-299)."""
    if warmup < 0 or iterations <= 0:
        raise ValueError("warmup must be non-negative and iterations must be positive")
    if dump_cuda is not None:
        raise ValueError("no CUDA source is generated: the kernel is precompiled for sm_100a")
    import torch

    from .engine import GroupedGemmPlan
    from . import _capi

    if not torch.cuda.is_available():
        raise RuntimeError("a CUDA-capable GPU is required; the engine has no CPU path")
    torch.backends.cuda.matmul.allow_tf32 = False
    descriptor = get_descriptor(version)
    dev = torch.device("cuda", torch.cuda.current_device())
    counts = list(plan.tokens_per_expert)
    total = sum(counts)

    # Inputs as the reference draws them (runner.py:136-171): device generator seeded
    # with the plan's seed, randn * 0.25, BF16; here packed expert-major.
    gen = torch.Generator(device=dev)
    gen.manual_seed(plan.seed)
    a = (torch.randn(max(1, total), spec.k, generator=gen, device=dev) * 0.25).to(torch.bfloat16)
    b = (torch.randn(spec.experts, spec.n, spec.k, generator=gen, device=dev) * 0.25) \
        .to(torch.bfloat16)
    d = torch.zeros(max(1, total), spec.n, dtype=torch.bfloat16, device=dev)

    engine_plan = GroupedGemmPlan()
    options = {**descriptor.engine_options(spec), **plan_options}
    status = engine_plan.initialize_packed(a, b, d, counts, **options)
    if status != _capi.OK:
        raise _capi.EngineError(status, f"bmoe_plan_initialize ({version})")
    stats = engine_plan.stats()

    def launch():
        rc = engine_plan.run()
        if rc != _capi.OK:
            raise _capi.EngineError(rc, "bmoe_plan_run")

    # correctness: per expert against A_e.float() @ B_e.float().T rounded to BF16, with
    # the reference's tolerances (runner.py:222-230)
    launch()
    status, report = engine_plan.poll()
    if status != _capi.OK:
        raise _capi.EngineError(status, f"device status (site {report.code})")
    max_abs = max_rel = 0.0
    row = 0
    for e, m in enumerate(counts):
        if not m:
            continue
        want = (a[row:row + m].float() @ b[e].float().T).to(torch.bfloat16)
        got = d[row:row + m]
        diff = (got.float() - want.float()).abs()
        max_abs = max(max_abs, float(diff.max().item()))
        max_rel = max(max_rel, float((diff / want.float().abs().clamp_min(1.0e-6)).max().item()))
        torch.testing.assert_close(got, want, rtol=2.0e-2, atol=5.0e-2)
        row += m

    timings: list[float] = []
    if not correctness_only:
        for _ in range(warmup):
            launch()
        torch.cuda.synchronize()
        starts = [torch.cuda.Event(enable_timing=True) for _ in range(iterations)]
        ends = [torch.cuda.Event(enable_timing=True) for _ in range(iterations)]
        for start, end in zip(starts, ends):
            # the queue re-arms itself at the end of every launch: nothing to reset here
            start.record()
            launch()
            end.record()
        torch.cuda.synchronize()
        timings = [s.elapsed_time(e) for s, e in zip(starts, ends)]
        status, report = engine_plan.poll()
        if status != _capi.OK:
            raise _capi.EngineError(status, f"device status (site {report.code})")

    median_ms = statistics.median(timings) if timings else math.nan
    features = routing_features(spec, plan)
    result = BenchmarkResult(
        device=torch.cuda.get_device_name(),
        implementation=descriptor.implementation,
        acquisition=descriptor.acquisition.replace(",", ";"),
        distribution=plan.distribution,
        experts=spec.experts,
        active_experts=plan.active_experts,
        tokens=spec.tokens,
        n=spec.n,
        k=spec.k,
        tiles=len(plan.tiles),
        ctas=int(stats.threadblock_count),
        pipe_depth=int(stats.stages),
        claim_size=spec.claim_size,
        hybrid_main_claim_size=spec.hybrid_main_claim_size,
        hybrid_tail_tiles=spec.hybrid_tail_tiles,
        cv_m=features.cv_m,
        max_over_mean_m=features.max_over_mean_m,
        inactive_expert_ratio=features.inactive_expert_ratio,
        small_m_expert_ratio=features.small_m_expert_ratio,
        expert_tile_cv=features.expert_tile_cv,
        max_expert_tiles_over_mean=features.max_expert_tiles_over_mean,
        tiles_per_cta=features.tiles_per_cta,
        useful_work_ratio=plan.useful_work_ratio,
        median_ms=median_ms,
        p95_ms=percentile_95(timings),
        effective_tflops=plan.logical_flops / (median_ms * 1.0e9) if timings else math.nan,
        max_abs_error=max_abs,
        max_rel_error=max_rel,
    )
    engine_plan.close()
    return result
