#!/usr/bin/env python
"""Benchmark of the MoE grouped-GEMM hot path on B200.

    python bench.py --gpus 1 --steps K --warmup W            # this engine
    python bench.py --impl reference ...                      # CPU reference arm

One "step" is one grouped GEMM over one routed batch. At one GPU the workload is
the Mixtral-8x7B-shaped up-projection (E=8, top-2, T=4096, K=4096, N=14336, Zipf
s=1.0 routing, seed 2026); with more GPUs it is the expert-parallel
DeepSeek-V3-shaped configuration (E=256, top-8, T=32768, K=7168, N=2048), one
rank per GPU, tokens exchanged by NCCL all-to-all. Inputs are synthetic
(A ~ N(0,1), W ~ N(0, 1/sqrt(K)), BF16). Prints ONE JSON line on rank 0.
"""

from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

WORKLOADS = {
    # name: experts, top_k, tokens, k, n, distribution id, zipf alpha, extra generator args
    "mixtral_e8_t4096_k4096_n14336_zipf1.0": dict(
        experts=8, top_k=2, tokens=4096, k=4096, n=14336, distribution=3, zipf_alpha=1.0),
    "cpu_runnable_e8_t256_k512_n1024_uniform": dict(
        experts=8, top_k=2, tokens=256, k=512, n=1024, distribution=0, zipf_alpha=1.2),
    # 8 experts take half of the assignments, the last 102 experts (40 %) are idle
    "deepseek_decode_e256_t256_k7168_n2048_heavy_sparse": dict(
        experts=256, top_k=8, tokens=256, k=7168, n=2048, distribution=4, zipf_alpha=1.2,
        heavy_fraction=8 / 256, heavy_share=0.5, inactive_fraction=0.4),
    "qwen3_e128_t16384_k2048_n768_zipf1.0": dict(
        experts=128, top_k=8, tokens=16384, k=2048, n=768, distribution=3, zipf_alpha=1.0),
    # half-size Mixtral-shaped case for profiler captures (weights 470 MB > L2)
    "profile_e8_t2048_k4096_n7168_zipf1.0": dict(
        experts=8, top_k=2, tokens=2048, k=4096, n=7168, distribution=3, zipf_alpha=1.0),
    # half-size decode-shaped case for profiler captures (weights 2.2 GB)
    "profile_decode_e128_t128_k7168_n2048_heavy_sparse": dict(
        experts=128, top_k=8, tokens=128, k=7168, n=2048, distribution=4, zipf_alpha=1.2,
        heavy_fraction=4 / 128, heavy_share=0.5, inactive_fraction=0.4),
    # one dense small-M problem (the weight-stream regime of the dense M-sweep)
    "profile_dense_m64_k2048_n7168": dict(
        experts=1, top_k=1, tokens=64, k=2048, n=7168, distribution=0, zipf_alpha=1.2),
    # small expert-parallel case for profiler captures of the routing kernels
    "profile_ep_e32_t4096_k7168_n2048_zipf1.0": dict(
        experts=32, top_k=4, tokens=4096, k=7168, n=2048, distribution=3, zipf_alpha=1.0),
    # same, top-8 and 16384 tokens: the weighted top-k sum reads 537 MB (> L2)
    "profile_ep_e32_t16384_top8_k7168_n2048_zipf1.0": dict(
        experts=32, top_k=8, tokens=16384, k=7168, n=2048, distribution=3, zipf_alpha=1.0),
    "ep_deepseek_e256_t32768_k7168_n2048_zipf1.0": dict(
        experts=256, top_k=8, tokens=32768, k=7168, n=2048, distribution=3, zipf_alpha=1.0),
}
# The reference's only published rows (its CUTLASS SM80 grouped baseline on one B200,
# docs/optimization_trajectory.md:14-22): E=64, 4096 routed rows, N=7168, K=2048, the
# library's default generator parameters; value = effective TFLOP/s at the median.
PUBLISHED_TFLOPS = {
    "published_e64_t4096_k2048_n7168_uniform": 221.247,
    "published_e64_t4096_k2048_n7168_heavy_hitter": 171.360,
    "published_e64_t4096_k2048_n7168_sparse": 304.694,
    "published_e64_t4096_k2048_n7168_zipf1.2": 174.681,
}
for _name, _dist, _alpha in (("uniform", 0, 1.2), ("heavy_hitter", 1, 1.2), ("sparse", 2, 1.2),
                             ("zipf1.2", 3, 1.2)):
    WORKLOADS["published_e64_t4096_k2048_n7168_" + _name] = dict(
        experts=64, top_k=1, tokens=4096, k=2048, n=7168, distribution=_dist, zipf_alpha=_alpha)
DEFAULT_WORKLOAD = "mixtral_e8_t4096_k4096_n14336_zipf1.0"
EP_WORKLOAD = "ep_deepseek_e256_t32768_k7168_n2048_zipf1.0"

# dram__bytes_read.sum + dram__bytes_write.sum per launch of the GEMM kernel, measured with
# ncu on the benchmarked configurations themselves (one launch each, DRAM counters and
# duration only) and on the small cases summarised under profiles/.
NCU_TRAFFIC_BYTES = {
    DEFAULT_WORKLOAD: 1242.6e6,                      # algorithmic 1241.5 MB
    "deepseek_decode_e256_t256_k7168_n2048_heavy_sparse": 4534.9e6,   # algorithmic 4529.8 MB
    "profile_e8_t2048_k4096_n7168_zipf1.0": 561.5e6,
    "profile_decode_e128_t128_k7168_n2048_heavy_sparse": 2283.9e6,
    "profile_dense_m64_k2048_n7168": 29.7e6,
}


def percentile(values, p):
    """sorted[ceil(p * n) - 1], the reference harness's rule
    (baselines/cutlass/benchmark.cu:133-138)."""
    s = sorted(values)
    idx = max(0, min(len(s) - 1, int(math.ceil(p * len(s)) - 1)))
    return s[idx]


def measured_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        data = json.loads(path.read_text())
        return {"source": "measured", "hbm_gbs": data["hbm_gbs"],
                "bf16_tflops": data["bf16_tflops"],
                "bf16_tflops_sustained": data.get("bf16_tflops_sustained")}
    return {"source": "fallback", "hbm_gbs": 6650.0, "bf16_tflops": 1590.0,
            "bf16_tflops_sustained": 1400.0}


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples during the timed region."""

    FIELDS = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.device_index = device_index
        self.proc = None
        self.path = None
        self.window = None   # (start, end) wall-clock seconds of the timed region

    def mark_region(self, start: float, end: float):
        """Host wall-clock bounds of the timed region: the median clock is taken over the
        samples inside it (the sampler also runs through the idle gaps around it)."""
        self.window = (start, end)

    @staticmethod
    def _seconds(stamp: str):
        import datetime

        try:
            return datetime.datetime.strptime(stamp, "%Y/%m/%d %H:%M:%S.%f").timestamp()
        except ValueError:
            return None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-i", str(self.device_index), "-lms", "20"],
                stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        clocks, reasons, power, stamps = [], set(), [], []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in Path(self.path).read_text().splitlines():
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                clocks.append(float(parts[1]))
                out["sm_max_mhz"] = float(parts[2])
                power.append(float(parts[3]))
                stamps.append(self._seconds(parts[0]))
            except ValueError:
                continue
            for name, flag in zip(names, parts[5:9]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.path)
        if clocks:
            # median over the samples taken inside the timed region (the sampler also runs
            # through the short idle gaps around it); all samples if none fall inside
            busy = []
            if self.window is not None:
                lo, hi = self.window
                busy = sorted(c for c, t in zip(clocks, stamps) if t is not None and lo <= t <= hi)
            if not busy:
                busy = sorted(clocks)
            out["sm_mhz"] = busy[len(busy) // 2]
            out["samples"] = len(clocks)
            out["samples_under_load"] = len(busy)
            out["power_w_max"] = max(power)
        out["reasons"] = sorted(reasons)
        return out


def workload_counts(engine, spec):
    """Routed rows per expert from the engine's (reference-exact) generator."""
    import ctypes as C

    cap = engine._capi
    cfg = cap.WorkloadConfig(
        experts=spec["experts"], distribution=spec["distribution"],
        total_tokens=spec["tokens"] * spec["top_k"], seed=2026,
        zipf_alpha=spec["zipf_alpha"],
        heavy_hitter_fraction=spec.get("heavy_fraction", 0.1),
        heavy_hitter_token_share=spec.get("heavy_share", 0.8),
        inactive_expert_fraction=spec.get("inactive_fraction", 0.5))
    out = (C.c_uint32 * spec["experts"])()
    cap.check(cap.load().bmoe_generate_workload(C.byref(cfg), out), "bmoe_generate_workload")
    return [int(x) for x in out]


def oracle_counts(lib, spec):
    """The same counts from the CPU oracle's restatement of the generator."""
    import ctypes as C

    import numpy as np

    out = np.zeros(spec["experts"], dtype=np.uint32)
    rc = lib.orc_generate_counts(
        C.c_uint32(spec["experts"]), C.c_uint64(spec["tokens"] * spec["top_k"]),
        C.c_uint32(spec["distribution"]), C.c_uint64(2026), C.c_double(spec["zipf_alpha"]),
        C.c_double(spec.get("heavy_fraction", 0.1)), C.c_double(spec.get("heavy_share", 0.8)),
        C.c_double(spec.get("inactive_fraction", 0.5)), out.ctypes.data_as(C.c_void_p))
    if rc != 0:
        raise RuntimeError("oracle generator rejected the workload")
    return [int(x) for x in out]


def synth_inputs(torch, counts, n, k, device):
    gen = torch.Generator(device=device).manual_seed(2026)
    total = sum(counts)
    a = torch.randn(total, k, generator=gen, device=device, dtype=torch.float32).to(torch.bfloat16)
    gen.manual_seed(2027)
    w = torch.empty(len(counts), n, k, device=device, dtype=torch.bfloat16)
    for e in range(len(counts)):
        w[e] = (torch.randn(n, k, generator=gen, device=device, dtype=torch.float32)
                * k ** -0.5).to(torch.bfloat16)
    return a, w


def bits(torch, t):
    import numpy as np

    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def load_oracle():
    import ctypes

    sys.path.insert(0, str(ROOT / "oracle"))
    import build_oracle

    lib = ctypes.CDLL(str(build_oracle.build_oracle()))
    lib.orc_grouped_gemm.restype = ctypes.c_uint64
    lib.orc_max_threads.restype = ctypes.c_int
    return lib


def host_threads() -> int:
    """Host threads the CPU arm may use (launchers such as torchrun export
    OMP_NUM_THREADS=1, which is not what this arm is meant to measure)."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def oracle_time(lib, a_bits, w_bits, counts, n, k, col_stride, col_phase=0):
    """Times the CPU restatement on every `col_stride`-th 128-column block of every
    expert, all rows (each sampled block costs what it costs in the full problem).
    Returns (output elements computed, seconds)."""
    import ctypes as C

    import numpy as np

    c = np.asarray(counts, dtype=np.uint32)
    d = np.zeros((a_bits.shape[0], n), dtype=np.uint16)
    lib.orc_grouped_gemm_column_sample.restype = C.c_uint64
    t0 = time.perf_counter()
    elements = lib.orc_grouped_gemm_column_sample(
        a_bits.ctypes.data_as(C.c_void_p), w_bits.ctypes.data_as(C.c_void_p),
        c.ctypes.data_as(C.c_void_p), C.c_uint32(len(c)), C.c_uint32(n), C.c_uint32(k),
        d.ctypes.data_as(C.c_void_p), C.c_uint32(col_stride), C.c_uint32(col_phase),
        C.c_int(host_threads()))
    dt = time.perf_counter() - t0
    return int(elements), dt


def column_stride_for(lib, a_bits, w_bits, counts, n, k, target_s):
    """Column-block stride whose sample takes about `target_s` seconds: calibrated on the
    thinnest sample (one block per expert)."""
    blocks = max(1, (n + 127) // 128)
    elements, dt = oracle_time(lib, a_bits, w_bits, counts, n, k, blocks)
    full_s = dt * blocks
    return max(1, min(blocks, int(math.ceil(full_s / max(target_s, 1e-3))))), blocks


def sample_text(stride, blocks, elements, total_elements, dt):
    return (f"every {stride}-th 128-column block of every expert, all rows "
            f"({elements / total_elements:.3f} of the output, {dt:.2f} s); "
            "FP32 sequential-k loop, OpenMP")


def cpu_sample(lib, a_bits, w_bits, counts, n, k, target_s=12.0):
    """Bounded CPU baseline: a column-block sample sized for about `target_s` seconds."""
    stride, blocks = column_stride_for(lib, a_bits, w_bits, counts, n, k, target_s)
    elements, dt = oracle_time(lib, a_bits, w_bits, counts, n, k, stride)
    tflops = 2.0 * elements * k / dt / 1e12
    return {"value": tflops, "unit": "TFLOP/s", "cores": host_threads(),
            "kind": "port",
            "sample": sample_text(stride, blocks, elements, sum(counts) * n, dt)}


def run_reference_arm(args, spec, workload):
    """The reference's CPU path for this op is the FP32 sequential-k loop of its
    tests (it ships no CPU GEMM runner); the oracle port of that loop is timed on
    all host cores, each step on a bounded column-block sample (the same kind of sample
    as the cpu_baseline leg of the engine line, so the two agree). The routing counts
    come from the oracle's own generator: nothing of the engine is loaded here."""
    import numpy as np

    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    lib = load_oracle()
    counts = oracle_counts(lib, spec)
    n, k = spec["n"], spec["k"]
    rng = np.random.default_rng(2026)
    total = sum(counts)

    def bf16_bits(x):  # round to nearest even, as the engine's inputs are made
        u = x.view(np.uint32)
        return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)

    # BF16 bit patterns of N(0,1) and N(0,1/sqrt(k)) samples.
    a_bits = bf16_bits(rng.standard_normal((total, k), dtype=np.float32))
    w_bits = np.empty((len(counts), n, k), dtype=np.uint16)
    for e in range(len(counts)):
        w_bits[e] = bf16_bits(rng.standard_normal((n, k), dtype=np.float32)
                              * np.float32(k ** -0.5))
    # Each step is one column-block sample of the workload, sized so that the whole run
    # (warm-up included) stays near 90 s of CPU time, at most 3 s per step.
    per_step_s = max(0.05, min(3.0, 90.0 / (args.steps + args.warmup)))
    stride, blocks = column_stride_for(lib, a_bits, w_bits, counts, n, k, per_step_s)
    for i in range(args.warmup):
        oracle_time(lib, a_bits, w_bits, counts, n, k, stride, i % stride)
    times, elements = [], 0
    for i in range(args.steps):
        done, dt = oracle_time(lib, a_bits, w_bits, counts, n, k, stride, i % stride)
        elements += done
        times.append(dt)
    per_step = sum(times) / len(times)
    tflops = 2.0 * elements * k / sum(times) / 1e12
    cores = host_threads()
    sample = sample_text(stride, blocks, elements // len(times), total * n, per_step) + \
        " per step, the block phase rotating"
    line = {
        "impl": "reference", "metric": "useful BF16 TFLOP/s per grouped GEMM",
        "value": tflops, "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": per_step * 1e3, "higher_is_better": True,
        "scaling": "strong" if args.gpus > 1 else "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": workload, "experts": spec["experts"], "top_k": spec["top_k"],
                   "tokens": spec["tokens"], "k": k, "n": n},
        "cpu_baseline": {"value": tflops, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                         "sample": sample},
        "e2e": {"value": tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def time_policy(torch, plan, stream, iters):
    """Per-launch CUDA-event samples (ms) of plan.run() on `stream`."""
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(iters)]
    stops = [torch.cuda.Event(enable_timing=True) for _ in range(iters)]
    for i in range(iters):
        starts[i].record(stream)
        status = plan.run(stream)
        stops[i].record(stream)
        if status != 0:
            raise RuntimeError(f"plan.run failed with status {status}")
    torch.cuda.synchronize()
    return [s.elapsed_time(e) for s, e in zip(starts, stops)]


def run_single_gpu(args, spec, workload):
    import torch

    import bmoe_b200 as engine

    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device; there is no CPU path for the engine")
    torch.cuda.set_device(0)
    dev = torch.device("cuda:0")
    stream = torch.cuda.current_stream()
    # the clock sampler needs a moment to come up: it starts before the inputs are made and
    # runs through the warm-up; the timed region's samples are picked by their time stamps
    sampler = ClockSampler(0)
    sampler.start()
    counts = workload_counts(engine, spec)
    n, k = spec["n"], spec["k"]
    total = sum(counts)
    flops = 2.0 * total * n * k
    a, w = synth_inputs(torch, counts, n, k, dev)
    fp8 = args.dtype == "fp8"
    if fp8:
        # E4M3 bit patterns of the same draws (weights x 8: out of the subnormal range);
        # operands are one byte per element, D stays BF16
        a = a.to(torch.float8_e4m3fn).view(torch.uint8)
        w8 = torch.empty(w.shape, dtype=torch.uint8, device=dev)
        for e in range(len(counts)):
            w8[e] = (w[e].float() * 8.0).to(torch.float8_e4m3fn).view(torch.uint8)
        w = w8
        del w8
    operand_bytes = 1 if fp8 else 2
    d = torch.zeros(total, n, dtype=torch.bfloat16, device=dev)
    active = sum(c > 0 for c in counts)
    algorithmic_bytes = operand_bytes * (total * k + active * n * k) + 2.0 * total * n

    def make_plan(policy, **opts):
        plan = engine.GroupedGemmPlan()
        status = plan.initialize_packed(a, w, d, counts, scheduler=policy, stream=stream, **opts)
        if status != 0:
            raise RuntimeError(f"initialize({policy}) -> {engine._capi.status_string(status)}")
        return plan

    def check(plan, what):
        status, rep = plan.poll()
        if status != 0:
            raise RuntimeError(f"{what}: {engine._capi.status_string(status)} "
                               f"(site {rep.code} cta {rep.cta} role {rep.role} tile {rep.tile})")

    # ---------------- headline: K timed steps of the chosen policy ----------
    plan = make_plan(args.policy, cta_group=args.cta_group)
    stats = plan.stats()
    load_start = time.time()   # the GPU is under this load from the first warm-up launch on
    for _ in range(args.warmup):
        plan.run(stream)
    check(plan, "warm-up")
    # the timed region: exactly K steps inside one event pair, right after the warm-up
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    launches_before = plan.stats().launches
    wall0 = time.time()
    t0.record(stream)
    for _ in range(args.steps):
        plan.run(stream)
    t1.record(stream)
    torch.cuda.synchronize()
    # clock samples: warm-up and timed region together (the region alone can be shorter than
    # one sampling interval at small K)
    sampler.mark_region(min(load_start, wall0), time.time())
    region_ms = t0.elapsed_time(t1)
    launches = plan.stats().launches - launches_before
    clocks = sampler.stop()
    # per-launch samples for p50 / p99 (at least 1000 launches for the p99), after the region;
    # clocks sampled again: this loop is long enough for the power cap to settle, and
    # nvidia-smi's clock reading lags behind a 0.15 s region
    loop_sampler = ClockSampler(0)
    loop_sampler.start()
    wall1 = time.time()
    samples = time_policy(torch, plan, stream, max(args.steps, args.sustained_launches))
    loop_sampler.mark_region(wall1 + 0.5 * (time.time() - wall1), time.time())
    clocks_sustained = loop_sampler.stop()
    check(plan, "timed region")
    ms_per_step = region_ms / args.steps
    value = flops / (ms_per_step * 1e-3) / 1e12
    avg_launch_ms = region_ms / args.steps   # average launch duration over the timed region

    # The same launch with the per-step set-up inside the measurement: counts upload,
    # worklist kernels and TMA descriptors rebuilt before every run (routing changes per step).
    replan = []
    for _ in range(60):
        r0, r1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        r0.record(stream)
        status = plan.initialize_packed(a, w, d, counts, scheduler=args.policy,
                                        cta_group=args.cta_group, stream=stream) or plan.run(stream)
        r1.record(stream)
        if status != 0:
            raise RuntimeError("re-plan step failed")
        replan.append((r0, r1))
    torch.cuda.synchronize()
    replan_ms = [x.elapsed_time(y) for x, y in replan][10:]
    check(plan, "re-plan steps")

    # ---------------- per-policy latency table (outside the headline region) --
    policies = {}
    if not args.no_policy_table:
        g = stats.cta_group
        table = [("expert_order", {}), ("static_persistent", {}), ("dynamic_queue", {}),
                 ("dynamic_queue", {"claim_size": 4}),
                 ("dynamic_queue", {"claim_size": 8, "hybrid_tail_tiles": 2 * 148 // g}),
                 ("compacted", {}), ("clc", {}), ("auto", {}),
                 ("expert_order", {"cta_group": 3 - g}), ("dynamic_queue", {"cta_group": 3 - g}),
                 ("clc", {"cta_group": 3 - g})]
        plans = []
        for policy, opts in table:
            label = policy
            if opts.get("claim_size"):
                label += "_c%d%s" % (opts["claim_size"],
                                     "_hybrid" if opts.get("hybrid_tail_tiles") else "")
            label += "_g%d" % opts.get("cta_group", g)
            plans.append((label, make_plan(policy, **{"cta_group": g, **opts})))
        for _ in range(max(3, args.warmup)):
            for _, p2 in plans:
                p2.run(stream)
        # Round-robin over the policies so that all of them see the same clock
        # and power state; one event pair per launch.
        iters = args.policy_iters
        ev = [[(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
               for _ in plans] for _ in range(iters)]
        torch.cuda.synchronize()
        for i in range(iters):
            for j, (_, p2) in enumerate(plans):
                ev[i][j][0].record(stream)
                p2.run(stream)
                ev[i][j][1].record(stream)
        torch.cuda.synchronize()
        for j, (label, p2) in enumerate(plans):
            check(p2, label)
            s = [ev[i][j][0].elapsed_time(ev[i][j][1]) for i in range(iters)]
            st = p2.stats()
            p50 = percentile(s, 0.5)
            policies[label] = {
                "p50_us": p50 * 1e3, "p99_us": percentile(s, 0.99) * 1e3,
                "min_us": min(s) * 1e3,
                "useful_tflops_p50": flops / (p50 * 1e-3) / 1e12,
                "ctas": st.threadblock_count, "resolved": st.resolved_scheduler,
                "claim_size": st.claim_size, "iters": len(s)}
            p2.close()
        base = policies["expert_order_g%d" % g]
        for label, row in policies.items():
            row["p99_speedup_vs_expert_order"] = base["p99_us"] / row["p99_us"]

    # ---------------- end to end through the public API, host buffers --------
    e2e, e2e_plan = None, None
    if not args.no_e2e:
        a_host = torch.empty(a.shape, dtype=a.dtype).pin_memory()
        a_host.copy_(a)
        d_host = torch.empty(d.shape, dtype=torch.bfloat16).pin_memory()
        # Two result buffers and two plans: while step i's D travels to the host on
        # a copy stream, step i+1 already uploads, re-plans and computes.
        e2e_plans = [engine.GroupedGemmPlan(), engine.GroupedGemmPlan()]
        e2e_plan = e2e_plans[0]
        d_pair = [d, torch.zeros_like(d)]
        copy_stream = torch.cuda.Stream()
        computed = [torch.cuda.Event(), torch.cuda.Event()]
        drained = [torch.cuda.Event(), torch.cuda.Event()]
        for ev in drained:
            ev.record(copy_stream)
        step_no = [0]

        def e2e_step():
            i = step_no[0] % 2
            step_no[0] += 1
            a.copy_(a_host, non_blocking=True)                      # H2D activations
            stream.wait_event(drained[i])                           # D[i] left the device
            status = e2e_plans[i].initialize_packed(a, w, d_pair[i], counts,
                                                    scheduler=args.policy,
                                                    cta_group=args.cta_group,
                                                    stream=stream)  # counts H2D, worklist, TMA maps
            status = status or e2e_plans[i].run(stream)
            computed[i].record(stream)
            with torch.cuda.stream(copy_stream):
                copy_stream.wait_event(computed[i])
                d_host.copy_(d_pair[i], non_blocking=True)          # D2H result
                drained[i].record(copy_stream)
            if status != 0:
                raise RuntimeError("e2e step failed")

        for _ in range(4):
            e2e_step()
        torch.cuda.synchronize()
        e2e_steps = max(4, min(args.steps, 20))
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(e2e_steps):
            e2e_step()
        stream.wait_stream(copy_stream)                             # the last D has arrived
        e1.record(stream)
        torch.cuda.synchronize()
        for p_ in e2e_plans:
            check(p_, "e2e")
        e2e_ms = e0.elapsed_time(e1) / e2e_steps
        e2e = {"value": flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
               "h2d_bytes_per_step": a_host.numel() * operand_bytes + 4 * len(counts)
               + 3 * 128 * len(counts) + 512,
               "d2h_bytes_per_step": d_host.numel() * 2, "ms_per_step": e2e_ms,
               "note": "weights stay resident on the device (plan state); every step uploads "
                       "activations and counts from pinned host memory, rebuilds the worklist "
                       "and TMA descriptors, computes, and returns D to pinned host memory; "
                       "the D2H copy of one step overlaps the next step (two D buffers)"}

    # ---------------- CPU baseline on a bounded sample ------------------------
    cpu = None
    if not args.no_cpu_baseline:
        lib = load_oracle()
        if fp8:
            # the oracle's FP8 definition: operands decoded exactly to BF16, then the same loop
            def decoded(t):
                import ctypes as C

                import numpy as np

                codes = np.ascontiguousarray(t.cpu().numpy())
                out = np.zeros(codes.shape, dtype=np.uint16)
                lib.orc_e4m3_to_bf16(codes.ctypes.data_as(C.c_void_p), C.c_uint64(codes.size),
                                     out.ctypes.data_as(C.c_void_p))
                return out
            cpu = cpu_sample(lib, decoded(a), decoded(w), counts, n, k, target_s=args.cpu_seconds)
        else:
            cpu = cpu_sample(lib, bits(torch, a), bits(torch, w), counts, n, k,
                             target_s=args.cpu_seconds)

    peaks = measured_peaks()
    achieved = flops / (avg_launch_ms * 1e-3) / 1e12
    # what a serving loop sees: the median of the long back-to-back loop, once the power
    # cap has settled the clocks
    sustained_ms = percentile(samples, 0.5)
    value_sustained = flops / (sustained_ms * 1e-3) / 1e12
    # FP8: no measured FP8 GEMM figure exists for this pool; the tensor pipe's FP8 rate is
    # nominally twice its BF16 rate, so the denominators are twice the measured BF16 ones
    tensor_scale = 2.0 if fp8 else 1.0
    tensor_peak = peaks["bf16_tflops"] * tensor_scale
    tensor_sustained = (peaks["bf16_tflops_sustained"] * tensor_scale
                        if peaks.get("bf16_tflops_sustained") else None)
    bound_is_tensor = flops / algorithmic_bytes > tensor_peak * 1e12 / (peaks["hbm_gbs"] * 1e9)
    if bound_is_tensor:
        roofline = {"bound": "tensor", "achieved": achieved, "peak": tensor_peak,
                    "unit": "TFLOP/s", "frac": achieved / tensor_peak,
                    # sustained loop against the sustained cuBLAS figure
                    "achieved_sustained": value_sustained,
                    "peak_sustained": tensor_sustained,
                    "frac_sustained": (value_sustained / tensor_sustained
                                       if tensor_sustained else None)}
    else:
        gbs = algorithmic_bytes / (avg_launch_ms * 1e-3) / 1e9
        gbs_sustained = algorithmic_bytes / (sustained_ms * 1e-3) / 1e9
        roofline = {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                    "frac": gbs / peaks["hbm_gbs"], "achieved_sustained": gbs_sustained,
                    "frac_sustained": gbs_sustained / peaks["hbm_gbs"]}
    roofline.update({"traffic": None if fp8 else NCU_TRAFFIC_BYTES.get(workload),
                     "peak_source": peaks["source"] + (
                         "; tensor peak = 2 x the measured BF16 figure (no FP8 measurement)"
                         if fp8 else ""),
                     "kernel": "grouped_gemm_kernel<%d, %s>" % (stats.tile_n, "pair" if stats.cta_group == 2 else "single"),
                     "algorithmic_flops_per_launch": flops,
                     "algorithmic_bytes_per_launch": algorithmic_bytes,
                     "avg_launch_ms": avg_launch_ms})

    line = {
        "metric": "useful %s TFLOP/s per grouped GEMM" % ("FP8" if fp8 else "BF16"),
        "value": value, "unit": "TFLOP/s",
        "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
        "higher_is_better": True, "scaling": "weak",
        # `value` is the K-step region right after the warm-up (a burst of a few ms at the
        # default K); `value_sustained` is the median launch of the long loop that follows
        "value_sustained": value_sustained, "sustained_launches": len(samples),
        "p50_us": percentile(samples, 0.5) * 1e3, "p99_us": percentile(samples, 0.99) * 1e3,
        "clocks": clocks, "clocks_sustained_loop": clocks_sustained,
        # value / the reference's published TFLOP/s, only where that exact row exists
        # (there the comparable figure is the median: useful_tflops_p50).
        "vs_baseline": (flops / (percentile(samples, 0.5) * 1e-3) / 1e12 / PUBLISHED_TFLOPS[workload]
                        if workload in PUBLISHED_TFLOPS and not fp8 else None),
        "dtype": "fp8_e4m3" if fp8 else "bf16", "data": "synthetic",
        "config": {"workload": workload, "experts": spec["experts"], "top_k": spec["top_k"],
                   "tokens": spec["tokens"], "k": k, "n": n, "policy": args.policy,
                   "resolved_policy": stats.resolved_scheduler,
                   "tile": [stats.tile_m, stats.tile_n, 128 if fp8 else 64],
                   "cta_group": stats.cta_group, "stages": stats.stages,
                   "ctas": stats.threadblock_count, "tiles": stats.total_tiles,
                   "l2": "weights (%.0f MB) exceed the 126 MB L2; no flush between steps"
                         % (active * n * k * operand_bytes / 1e6)},
        "latency_samples": len(samples),
        "p50_us_with_replan": percentile(replan_ms, 0.5) * 1e3,
        "p99_us_with_replan": percentile(replan_ms, 0.99) * 1e3,
        "policies": policies, "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e,
        "gpu_launches": launches,
    }
    if e2e is not None:
        e2e["note"] += ("; the step time is the D2H copy of D over PCIe (%.0f MB per step), "
                        "the GPU part is %.2f ms" % (d.numel() * 2 / 1e6, sustained_ms))
    plan.close()
    if e2e_plan is not None:
        for p_ in e2e_plans:
            p_.close()
    print(json.dumps(line), flush=True)


def run_skew_sweep(args):
    """Qwen3-MoE-shaped skew sweep (E=128, top-8, T=16384, K=2048, N=768): per routing
    point the reference's workload / schedule-model metrics, the variant its threshold
    rule picks, and the engine's p50 / p99 per policy. One JSON line with a "sweep" list."""
    import ctypes as C

    import torch

    import bmoe_b200 as engine

    cap = engine._capi
    lib = cap.load()
    torch.cuda.set_device(0)
    dev = torch.device("cuda:0")
    stream = torch.cuda.current_stream()
    base = dict(experts=128, top_k=8, tokens=16384, k=2048, n=768)
    points = [(label, dict(base, distribution=dist_id, zipf_alpha=alpha))
              for label, dist_id, alpha in (("uniform", 0, 1.2), ("zipf0.5", 3, 0.5),
                                            ("zipf1.0", 3, 1.0), ("zipf1.5", 3, 1.5))]
    if args.sweep_all:
        # the other single-GPU configurations, for the p99-vs-expert-order table
        points += [("mixtral_zipf1.0", WORKLOADS[DEFAULT_WORKLOAD]),
                   ("decode_heavy_sparse",
                    WORKLOADS["deepseek_decode_e256_t256_k7168_n2048_heavy_sparse"]),
                   ("cpu_runnable_uniform", WORKLOADS["cpu_runnable_e8_t256_k512_n1024_uniform"])]
        points += [(name, WORKLOADS[name]) for name in sorted(PUBLISHED_TFLOPS)]
    out = []
    for label, spec in points:
        counts = workload_counts(engine, spec)
        n, k = spec["n"], spec["k"]
        arr = (C.c_uint32 * len(counts))(*counts)
        wm = cap.WorkloadMetrics()
        lib.bmoe_workload_metrics_compute(arr, len(counts), n, 128, 128, C.byref(wm))
        model = {}
        for name, sched in (("expert_order", 0), ("static_persistent", 1), ("dynamic_queue", 2)):
            sm = cap.ScheduleMetrics()
            lib.bmoe_host_simulate(sched, arr, len(counts), n, 128, 128, 148, None, 0, None,
                                   C.byref(sm))
            model[name] = {"tail_ratio": sm.tail_ratio, "cta_work_cv": sm.cta_work_cv,
                           "useful_work_ratio": sm.useful_work_ratio}
        feats = cap.RoutingFeatures()
        lib.bmoe_routing_features_compute(arr, len(counts), n, 128, 128, 148, C.byref(feats))
        variant = C.c_uint32(0)
        lib.bmoe_select_variant(C.byref(feats), None, C.byref(variant))
        a, w = synth_inputs(torch, counts, n, k, dev)
        d = torch.zeros(sum(counts), n, dtype=torch.bfloat16, device=dev)
        flops = 2.0 * sum(counts) * n * k
        plans = []
        # "auto" = the plan's own rule (fitted thresholds); "reference_rule" = the variant
        # the reference's bootstrap thresholds pick, launched as that variant.
        picked = cap.VARIANT_NAMES[variant.value]
        mspec = engine.MoESpec(experts=len(counts), tokens=sum(counts), n=n, k=k)
        ref_opts = dict(engine.get_descriptor(picked).engine_options(mspec))
        ref_policy = ref_opts.pop("scheduler")
        ref_opts.pop("cta_count", None)
        for label_, policy, opts in (("expert_order", "expert_order", {}),
                                     ("static_persistent", "static_persistent", {}),
                                     ("dynamic_queue", "dynamic_queue", {}), ("clc", "clc", {}),
                                     ("auto", "auto", {}),
                                     ("reference_rule", ref_policy, ref_opts),
                                     ("expert_order_g1", "expert_order", {"cta_group": 1}),
                                     ("dynamic_queue_g1", "dynamic_queue", {"cta_group": 1}),
                                     ("clc_g1", "clc", {"cta_group": 1}),
                                     ("expert_order_g2", "expert_order", {"cta_group": 2}),
                                     ("dynamic_queue_g2", "dynamic_queue", {"cta_group": 2}),
                                     ("clc_g2", "clc", {"cta_group": 2})):
            plan = engine.GroupedGemmPlan()
            cap.check(plan.initialize_packed(a, w, d, counts, scheduler=policy, stream=stream,
                                             **{"cta_group": args.cta_group, **opts}), label_)
            plans.append((label_, plan))
        for _ in range(max(3, args.warmup)):
            for _, plan in plans:
                plan.run(stream)
        iters = args.policy_iters
        ev = [[(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
               for _ in plans] for _ in range(iters)]
        torch.cuda.synchronize()
        for i in range(iters):
            for j, (_, plan) in enumerate(plans):
                ev[i][j][0].record(stream)
                plan.run(stream)
                ev[i][j][1].record(stream)
        torch.cuda.synchronize()
        timing = {}
        for j, (policy, plan) in enumerate(plans):
            status, _ = plan.poll()
            if status != 0:
                raise RuntimeError(f"{policy}: {cap.status_string(status)}")
            ms = [ev[i][j][0].elapsed_time(ev[i][j][1]) for i in range(iters)]
            p50 = percentile(ms, 0.5)
            st_ = plan.stats()
            timing[policy] = {"p50_us": p50 * 1e3, "p99_us": percentile(ms, 0.99) * 1e3,
                              "useful_tflops_p50": flops / (p50 * 1e-3) / 1e12,
                              "cta_group": st_.cta_group, "tile_n": st_.tile_n,
                              "resolved": st_.resolved_scheduler, "ctas": st_.threadblock_count}
            plan.close()
        for row in timing.values():
            row["p99_speedup_vs_expert_order"] = timing["expert_order"]["p99_us"] / row["p99_us"]
        best = min(timing, key=lambda name: timing[name]["p50_us"])
        auto_gap = timing["auto"]["p50_us"] / timing[best]["p50_us"] - 1.0
        out.append({"routing": label, "shape": {"experts": spec["experts"], "rows": sum(counts),
                                                 "k": k, "n": n},
                    "cv_m": wm.coefficient_of_variation,
                    "max_over_mean_m": wm.max_over_mean, "tile_count_cv": wm.tile_count_cv,
                    "small_m_expert_ratio": wm.small_m_expert_ratio,
                    "total_tiles_128x128": wm.total_tiles, "schedule_model_148_ctas": model,
                    "reference_rule_picks": cap.VARIANT_NAMES[variant.value],
                    "best_p50": best, "auto_p50_over_best": auto_gap,
                    "engine": timing})
        del a, w, d
    print(json.dumps({"metric": "p50/p99 us per grouped GEMM vs routing skew", "unit": "us",
                      "n_gpus": 1, "dtype": "bf16", "data": "synthetic",
                      "config": {"workload": "qwen3_skew_sweep_e128_t16384_k2048_n768", **base},
                      "iters": args.policy_iters, "sweep": out}), flush=True)


def run_dense_sweep(args):
    """Dense M-sweep at N=7168, K=2048 (docs/sm100_native_dense.md:124-128 and
    tools/run_b200_optimization_suite.sh:66-73 of the reference). All three columns come
    from the reference's OWN benchmark program (benchmarks/sm100_dense_benchmark.cu /
    sm100_2sm_benchmark.cu, unmodified: 20 warm-up launches, 200 timed with one CUDA-event
    pair each, median): linked against this engine's drop-in dense plans (single CTA and
    CTA pair), and linked against the reference's own sm_100a kernel, its CUTLASS 1-SM
    collective (src/kernels/sm100_dense_gemm.cu). One JSON line with a "sweep" list."""
    n, k = 7168, 2048
    peaks = measured_peaks()
    bin_dir = ROOT / "oracle" / "_ref" / "bin"
    programs = {"engine_single_cta": bin_dir / "ref_sm100_dense_benchmark",
                "engine_cta_pair": bin_dir / "ref_sm100_2sm_benchmark",
                "reference_cutlass_1sm": bin_dir / "ref_native_sm100_dense_benchmark"}
    missing = [str(p.relative_to(ROOT)) for p in programs.values() if not p.exists()]

    def one(program, m):
        proc = subprocess.run([str(program), f"--m={m}", f"--n={n}", f"--k={k}",
                               "--warmup=20", "--iterations=200", "--csv"],
                              capture_output=True, text=True, timeout=300)
        lines = proc.stdout.strip().splitlines()
        if proc.returncode != 0 or len(lines) < 2:
            return {"unavailable": (proc.stderr.strip() or proc.stdout.strip())[-200:]}
        rec = dict(zip(lines[0].split(","), lines[-1].split(",")))
        return {"median_us": float(rec["median_ms"]) * 1e3, "p95_us": float(rec["p95_ms"]) * 1e3,
                "tflops": float(rec["tflops"]), "kernel": rec["kernel"],
                "tile": [int(rec["tile_m"]), int(rec["tile_n"]), int(rec["tile_k"])],
                "ctas": int(rec["persistent_ctas"])}

    rows = []
    for m in (16, 32, 64, 128, 256, 512, 1024, 4096, 8192):
        flops = 2.0 * m * n * k
        algorithmic_bytes = 2.0 * (m * k + n * k + m * n)
        floor_us = max(algorithmic_bytes / (peaks["hbm_gbs"] * 1e9),
                       flops / (peaks["bf16_tflops"] * 1e12)) * 1e6
        row = {"m": m, "roofline_floor_us": floor_us}
        for label, program in programs.items():
            row[label] = one(program, m) if program.exists() else {"unavailable": "not built"}
        mine = [row[x]["median_us"] for x in ("engine_single_cta", "engine_cta_pair")
                if "median_us" in row[x]]
        if mine:
            row["engine_best_us"] = min(mine)
            row["engine_best_over_floor"] = min(mine) / floor_us
            if "median_us" in row["reference_cutlass_1sm"]:
                row["speedup_vs_reference"] = row["reference_cutlass_1sm"]["median_us"] / min(mine)
        rows.append(row)
    print(json.dumps({"metric": "median us per dense GEMM vs M (N=7168, K=2048)", "unit": "us",
                      "n_gpus": 1, "dtype": "bf16", "data": "synthetic",
                      "config": {"workload": "dense_sweep_n7168_k2048", "n": n, "k": k,
                                 "warmup": 20, "iterations": 200,
                                 "harness": "the reference's benchmark programs, unmodified"},
                      "reference_arm": ("unavailable: not built: " + ", ".join(missing)) if missing
                      else "the reference's CUTLASS 1-SM collective (cluster 1x1x1), unmodified "
                           "sources, CUTLASS 4.5.0 headers found in site-packages (the "
                           "reference pins 4.6.0)",
                      "sweep": rows}), flush=True)


def run_dense_timeline(args):
    """Where the time of a small dense launch goes: the per-CTA wait accounting and time line
    (bmoe_plan_set_trace, 16 words per CTA, SM cycles) of one launch after warm-up, median
    over the CTAs, for the small-M points of the dense sweep and a one-tile problem; beside
    each the median of 200 event pairs around single launches. One JSON line."""
    import numpy as np
    import torch

    import bmoe_b200 as engine

    dev = torch.device("cuda:0")
    torch.cuda.set_device(0)
    stream = torch.cuda.current_stream()
    words = ["producer_wait_info", "producer_wait_stage", "mma_wait_info", "mma_wait_accumulator",
             "mma_wait_operands", "epilogue_wait_info", "epilogue_wait_accumulator",
             "epilogue_drain", "tiles", "kernel", "mma_issue", "t_setup_done",
             "t_first_operands", "t_last_mma_issued", "t_last_accumulator", "t_epilogue_done"]
    gen = torch.Generator(device=dev).manual_seed(1)
    rows = []
    for m, n, k in ((16, 128, 64), (128, 7168, 64), (64, 7168, 2048), (128, 7168, 2048),
                    (256, 7168, 2048)):
        w = (torch.randn(1, n, k, generator=gen, device=dev) * k ** -0.5).to(torch.bfloat16)
        a = torch.randn(m, k, generator=gen, device=dev).to(torch.bfloat16)
        d = torch.zeros(m, n, dtype=torch.bfloat16, device=dev)
        plan = engine.GroupedGemmPlan()
        status = plan.initialize_packed(a, w, d, [m], scheduler="expert_order", cta_group=1,
                                        tile_n=128, stream=stream)
        if status != 0:
            raise RuntimeError(engine._capi.status_string(status))
        for _ in range(20):
            plan.run(stream)
        pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
                 for _ in range(200)]
        torch.cuda.synchronize()
        for e0, e1 in pairs:
            e0.record(stream)
            plan.run(stream)
            e1.record(stream)
        torch.cuda.synchronize()
        stats = plan.stats()
        trace = torch.zeros(stats.threadblock_count, 16, dtype=torch.int64, device=dev)
        plan.set_trace(trace)
        plan.run(stream)
        status, _ = plan.poll()
        if status != 0:
            raise RuntimeError(engine._capi.status_string(status))
        plan.set_trace(None)
        t = trace.cpu().numpy().astype(np.float64)
        rows.append({"m": m, "n": n, "k": k, "ctas": stats.threadblock_count,
                     "tile": [stats.tile_m, stats.tile_n, 64], "k_blocks": (k + 63) // 64,
                     "event_pair_median_us": percentile([x.elapsed_time(y) for x, y in pairs],
                                                        0.5) * 1e3,
                     "cycles_median_over_ctas": {name: float(np.median(t[:, i]))
                                                 for i, name in enumerate(words)}})
        plan.close()
    print(json.dumps({"metric": "CTA time line of small dense launches", "unit": "SM cycles",
                      "n_gpus": 1, "dtype": "bf16", "data": "synthetic",
                      "config": {"workload": "dense_timeline_tile128x128"}, "rows": rows}),
          flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="engine", choices=["engine", "reference"])
    ap.add_argument("--workload", default=None, choices=sorted(WORKLOADS))
    # "auto" = the engine's own fitted rule (launch control on the headline workload);
    # every explicit policy is in the table.
    ap.add_argument("--policy", default="auto")
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp8"],
                    help="operand type of the single-GPU run: bf16 (the reference's contract) "
                         "or fp8 (E4M3 operands, an engine extension; D stays BF16)")
    ap.add_argument("--cta-group", type=int, default=0, choices=[0, 1, 2],
                    help="0 = engine picks per routing (default)")
    ap.add_argument("--policy-iters", type=int, default=1000,
                    help="launches per policy in the latency table (p99 needs >= 1000)")
    ap.add_argument("--sustained-launches", type=int, default=1000,
                    help="back-to-back launches of the loop behind value_sustained / p50 / p99")
    ap.add_argument("--no-policy-table", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-single-gpu-ref", action="store_true")
    ap.add_argument("--exchange", default="fused", choices=["fused", "peer", "nccl"],
                    help="multi-GPU token exchange: fused = peer-memory pushes overlapped with "
                         "the gated grouped GEMM; peer = two routing kernels with barriers; "
                         "nccl = all-to-all with local re-packing")
    ap.add_argument("--ep-groups", type=int, default=0,
                    help="expert groups overlapped between exchange and GEMM (multi-GPU); "
                         "0 = 8 for the fused exchange, 1 otherwise")
    ap.add_argument("--comm-sms", type=int, default=8,
                    help="SMs the pipelined GEMM leaves to the exchange kernels")
    ap.add_argument("--dispatch-ctas", type=int, default=0,
                    help="fused exchange: CTAs of the remote-row kernel (0 = one per SM)")
    ap.add_argument("--exchange-sms", type=int, default=-1,
                    help="fused exchange: SMs the GEMM leaves to the remote-row kernel "
                         "(0 = share SMs, see --dispatch-ctas; -1 = 16)")
    ap.add_argument("--copy-engine-kb", type=int, default=0,
                    help="fused exchange: (expert, source) blocks of at least this many KiB "
                         "travel as peer copies issued by the host (copy engines) instead of "
                         "SM stores; 0 = all rows through the SMs")
    ap.add_argument("--send-once", type=int, default=-1, choices=[-1, 0, 1],
                    help="fused exchange: a token routed to several experts of one other rank "
                         "crosses NVLink once and the owner's GEMM kernel copies the row onto "
                         "the other packed rows (-1 = off)")
    ap.add_argument("--split-hot", action="store_true",
                    help="fused exchange: cut experts above half a rank's fair share of the "
                         "tiles into row shards placed on several ranks")
    ap.add_argument("--bulk-copies", action="store_true",
                    help="fused exchange: remote rows as TMA bulk copies through shared memory")
    ap.add_argument("--no-push", action="store_true",
                    help="fused exchange: return result rows with a kernel after the GEMM "
                         "instead of from its epilogue")
    ap.add_argument("--topk-weights", action="store_true",
                    help="expert-parallel arm: finish with the weighted top-k sum (y is [tokens, n])")
    ap.add_argument("--cpu-seconds", type=float, default=12.0)
    ap.add_argument("--sweep", action="store_true",
                    help="run the Qwen3-shaped routing-skew sweep instead of the headline")
    ap.add_argument("--sweep-all", action="store_true",
                    help="with --sweep: add the Mixtral-shaped and the decode-shaped "
                         "configurations to the routing points")
    ap.add_argument("--dense-sweep", action="store_true",
                    help="dense M-sweep (N=7168, K=2048): engine dense plans next to the "
                         "reference's own CUTLASS 1-SM kernel")
    ap.add_argument("--dense-timeline", action="store_true",
                    help="wait accounting and CTA time line of small dense launches")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.dense_timeline:
        run_dense_timeline(args)
        return
    if args.sweep:
        run_skew_sweep(args)
        return
    if args.dense_sweep:
        run_dense_sweep(args)
        return
    workload = args.workload or (DEFAULT_WORKLOAD if args.gpus == 1 else EP_WORKLOAD)
    spec = WORKLOADS[workload]
    if args.impl == "reference":
        if args.dtype != "bf16":
            raise SystemExit("--impl reference times the reference's BF16 contract only")
        run_reference_arm(args, spec, workload)
        return
    single = args.gpus == 1 and int(os.environ.get("WORLD_SIZE", "1")) == 1
    if single and not workload.startswith(("ep_", "profile_ep_")):
        run_single_gpu(args, spec, workload)
    else:
        if args.dtype != "bf16":
            raise SystemExit("--dtype fp8 is a single-GPU option: the expert-parallel exchange "
                             "moves BF16 rows")
        import ep_bench  # the multi-GPU arm, beside this file

        ep_bench.run(args, spec, workload)


if __name__ == "__main__":
    # Standard output carries exactly one JSON line. Libraries that write to file
    # descriptor 1 themselves (NCCL's version banner) are sent to stderr: Python's
    # sys.stdout keeps the real stdout, descriptor 1 becomes a copy of stderr.
    sys.stdout.flush()
    sys.stdout = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)
    main()
    sys.stdout.flush()
