"""Multi-GPU arm of bench.py (a benchmark driver, not part of the package): the
expert-parallel configuration.

E=256 experts, top-8, T tokens split evenly across ranks, K=7168, N=2048, BF16,
Zipf s=1.0 routing (seeded multinomial without replacement per token). Experts are
placed by tile-count balance once; every step runs counts exchange, dispatch
all-to-all, local grouped GEMM and combine all-to-all. Timed on the device with
CUDA events, maximum over ranks; total work is fixed as ranks grow (strong scaling).
Outside the timed region every rank's result rows are compared, bit for bit, with the
same workload computed by the single-GPU engine on rank 0; a mismatch fails the run.
"""

from __future__ import annotations

import json
import os
import time


def _routing(torch, spec):
    """Global per-token expert ids, identical on every rank (CPU generator)."""
    gen = torch.Generator().manual_seed(2026)
    experts = spec["experts"]
    weights = 1.0 / torch.arange(1, experts + 1, dtype=torch.float64) ** spec["zipf_alpha"]
    if spec["distribution"] == 0:
        weights = torch.ones(experts, dtype=torch.float64)
    return torch.multinomial(weights.expand(spec["tokens"], -1), spec["top_k"],
                             replacement=False, generator=gen)


def _expert_weights(torch, expert_ids, n, k, dev):
    w = torch.empty(len(expert_ids), n, k, dtype=torch.bfloat16, device=dev)
    gen = torch.Generator(device=dev)
    for i, e in enumerate(expert_ids):
        gen.manual_seed(2027 + int(e))
        w[i] = (torch.randn(n, k, generator=gen, device=dev, dtype=torch.float32)
                * k ** -0.5).to(torch.bfloat16)
    return w


def run(args, spec, workload):
    import torch
    import torch.distributed as dist

    import bmoe_b200 as engine
    from bmoe_b200 import ep

    import bench  # percentile, ClockSampler, measured_peaks

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("the expert-parallel bench needs CUDA devices")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        # keep stdout to the one JSON line (NCCL_DEBUG=VERSION prints a banner there)
        if os.environ.get("NCCL_DEBUG", "").upper() in ("", "VERSION"):
            os.environ["NCCL_DEBUG"] = "WARN"
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(value: float) -> float:
        if world == 1:
            return value
        t = torch.tensor([value], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # the clock sampler needs a moment to come up: it starts before the set-up and runs
    # through the warm-up; the timed region's samples are picked by their time stamps
    sampler = bench.ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    n, k, top_k, tokens = spec["n"], spec["k"], spec["top_k"], spec["tokens"]
    ids_all = _routing(torch, spec)
    global_counts = torch.bincount(ids_all.reshape(-1), minlength=spec["experts"]).tolist()
    place_tile_m = 256 if args.cta_group != 1 else 128
    parts = None
    if args.exchange == "fused" and world > 1 and args.split_hot:
        # experts above half a rank's fair share of the tiles are cut into row shards
        parts, owner, rank_tiles = ep.split_and_place_experts(global_counts, world, n,
                                                              tile_m=place_tile_m, tile_n=256)
    else:
        owner, rank_tiles = ep.place_experts(global_counts, world, n, tile_m=place_tile_m,
                                             tile_n=256)
    lo, hi = tokens * rank // world, tokens * (rank + 1) // world
    ids_local = ids_all[lo:hi].to(dev)
    gen = torch.Generator(device=dev).manual_seed(4000 + rank)
    x_local = torch.randn(hi - lo, k, generator=gen, device=dev,
                          dtype=torch.float32).to(torch.bfloat16)
    ep_groups = args.ep_groups or (8 if args.exchange == "fused" else 1)
    groups = ep_groups if world > 1 else 1
    gates = None
    if args.topk_weights:
        # router gates: the last step becomes the weighted top-k sum, y is [tokens, n]
        gates = torch.softmax(torch.randn(hi - lo, top_k, generator=gen, device=dev), dim=1)
        groups = 1
    extra = {"topk_weights": gates} if gates is not None else {}
    plan_options = {"cta_group": args.cta_group}
    if groups > 1 and args.comm_sms > 0:
        # Leave a few SMs to the exchange kernels that run beside the GEMM.
        sms = torch.cuda.get_device_properties(dev).multi_processor_count
        pair = args.cta_group != 1
        plan_options = {"cta_group": 2 if pair else 1,
                        "cta_count": max(1, (sms - args.comm_sms) // (2 if pair else 1))}
    # The overlapped exchange needs a persistent grid (it keeps SMs free for the pushes and
    # plans the step on the device): "auto" means the claim-1 queue here.
    fused_policy = "dynamic_queue" if args.policy == "auto" else args.policy
    # Defaults of the overlapped exchange: 16 SMs set aside for the pushes, every
    # assignment sends its own row. The send-once exchange (--send-once 1) cuts the NVLink
    # bytes 1.4-4x; at two and four GPUs, where the gated GEMM and not the pushes bounds the
    # step, it changed the step by less than the run-to-run spread (3 %), with SMs set aside
    # or shared.
    send_once = max(0, args.send_once)
    exchange_sms = args.exchange_sms if args.exchange_sms >= 0 else 16
    if args.exchange == "fused":
        from bmoe_b200 import ep_fused

        layer = ep_fused.FusedExpertParallelLayer(
            owner, n, k, rank=rank, world=world, rows_cap=tokens * top_k,
            assignments_cap=(hi - lo) * top_k, scheduler=fused_policy,
            exchange_groups=ep_groups, cta_group=args.cta_group,
            dispatch_ctas=args.dispatch_ctas, push_results=not args.no_push,
            exchange_sms=exchange_sms, expert_parts=parts,
            bulk_copies=args.bulk_copies, copy_engine_min_bytes=args.copy_engine_kb * 1024,
            send_once=bool(send_once))
        ops = layer
        plain = layer
        groups = layer.groups
    elif args.exchange == "peer":
        from bmoe_b200 import ep_peer

        # Row capacity: every assignment of the batch could land on one rank.
        layer = ep_peer.PeerExpertParallelLayer(
            owner, n, k, rank=rank, world=world, rows_cap=tokens * top_k,
            scheduler=args.policy, cta_group=args.cta_group)
        ops = layer          # launches / poll live on the layer
        plain = layer
        groups = 1
    else:
        ops = ep.CudaOps(scheduler=args.policy, **plan_options)
        layer = ep.ExpertParallelLayer(owner, n, k, rank=rank, world=world, ops=ops,
                                       pipeline_groups=groups)
        # un-pipelined twin for the per-phase split
        plain = layer if groups == 1 else ep.ExpertParallelLayer(
            owner, n, k, rank=rank, world=world,
            ops=ep.CudaOps(scheduler=args.policy, cta_group=args.cta_group))
    exchange_sms_used = getattr(layer, "exchange_sms", 0)
    layer_info = type("LayerInfo", (), {"device_plan": getattr(layer, "device_plan", False),
                                        "send_once": getattr(layer, "send_once", False)})
    copy_bytes = 0
    w_local = _expert_weights(torch, layer.local_experts, n, k, dev)
    total_flops = 2.0 * tokens * top_k * n * k
    stream = torch.cuda.current_stream()

    for _ in range(args.warmup):
        layer.forward(x_local, ids_local, w_local, **extra)
    ops.poll()
    barrier()
    launches_before = ops.launches
    barrier()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    wall0 = time.time()
    t0.record(stream)
    for _ in range(args.steps):
        layer.forward(x_local, ids_local, w_local, **extra)
    t1.record(stream)
    barrier()
    sampler.mark_region(wall0, time.time())
    ms_per_step = max_over_ranks(t0.elapsed_time(t1) / args.steps)
    launches = ops.launches - launches_before
    copy_bytes = getattr(layer, "copy_bytes", 0)
    clocks = sampler.stop() if rank == 0 else None
    ops.poll()

    # per-phase split and per-step samples (separate short loop)
    phase_sum, step_samples = {}, []
    phase_iters = max(3, min(args.steps, 20))
    for _ in range(phase_iters):
        barrier()
        plain.forward(x_local, ids_local, w_local, record_events=True, **extra)
        phases = plain.phase_times_ms()
        step_samples.append(max_over_ranks(sum(v for key, v in phases.items()
                                                if not key.endswith("_overlapped"))))
        for name, ms in phases.items():
            phase_sum[name] = phase_sum.get(name, 0.0) + ms
    phases_ms = {name: max_over_ranks(v / phase_iters) for name, v in phase_sum.items()}
    local_rows = sum(plain.last_local_m)
    gemm_flops_local = 2.0 * local_rows * n * k
    gemm_ms_local = phase_sum["gemm"] / phase_iters
    rows_max = max_over_ranks(float(local_rows))

    # end to end: activations from pinned host memory, result back to the host
    x_host = torch.empty(x_local.shape, dtype=torch.bfloat16).pin_memory()
    x_host.copy_(x_local)
    y_host = torch.empty((hi - lo) * (1 if gates is not None else top_k), n,
                         dtype=torch.bfloat16).pin_memory()
    e2e_steps = max(3, min(args.steps, 10))

    def e2e_step():
        x_local.copy_(x_host, non_blocking=True)
        y = layer.forward(x_local, ids_local, w_local, **extra)
        y_host.copy_(y, non_blocking=True)

    for _ in range(2):
        e2e_step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(e2e_steps):
        e2e_step()
    e1.record(stream)
    barrier()
    e2e_ms = max_over_ranks(e0.elapsed_time(e1) / e2e_steps)
    ops.poll()
    # this rank's result rows of one more step, kept for the parity check below
    y_ep = layer.forward(x_local, ids_local, w_local, **extra).clone()
    ops.poll()

    # The same workload on ONE GPU (rank 0 alone, no exchange), so that strong
    # scaling can be read from a single run.
    single_gpu = None
    parity = None
    if world > 1 and not args.no_single_gpu_ref:
        # Every rank's token rows (and router gates) travel to rank 0, which runs the whole
        # batch through the single-GPU engine; each rank then receives the rows that belong
        # to its tokens and compares them with what the expert-parallel step gave it.
        per_rank = (hi - lo)
        even = tokens % world == 0
        x_parts = [torch.empty_like(x_local) for _ in range(world)] if rank == 0 and even else None
        g_parts = None
        if even:
            dist.gather(x_local, x_parts, dst=0)
            if gates is not None:
                g_parts = [torch.empty_like(gates) for _ in range(world)] if rank == 0 else None
                dist.gather(gates, g_parts, dst=0)
        y_ref_parts = None
        if rank == 0:
            del w_local, layer, ops, plain
            torch.cuda.empty_cache()
            solo_owner = [0] * spec["experts"]
            solo_ops = ep.CudaOps(scheduler=args.policy, cta_group=args.cta_group)
            solo = ep.ExpertParallelLayer(solo_owner, n, k, rank=0, world=1, ops=solo_ops)
            w_all = _expert_weights(torch, list(range(spec["experts"])), n, k, dev)
            if even:
                x_all = torch.cat(x_parts, dim=0)
                del x_parts
            else:
                gen.manual_seed(4000)
                x_all = torch.randn(tokens, k, generator=gen, device=dev,
                                    dtype=torch.float32).to(torch.bfloat16)
            solo_extra = ({"topk_weights": torch.cat(g_parts, dim=0)}
                          if gates is not None and even else {})
            ids_dev = ids_all.to(dev)
            for _ in range(3):
                solo.forward(x_all, ids_dev, w_all, **solo_extra)
            torch.cuda.synchronize()
            s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            solo_steps = max(3, min(args.steps, 10))
            s0.record(stream)
            for _ in range(solo_steps):
                y_all = solo.forward(x_all, ids_dev, w_all, **solo_extra)
            s1.record(stream)
            torch.cuda.synchronize()
            solo_ops.poll()
            solo_ms = s0.elapsed_time(s1) / solo_steps
            single_gpu = {"value": total_flops / (solo_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                          "ms_per_step": solo_ms, "steps": solo_steps}
            if even:
                y_ref_parts = list(y_all.reshape(world, -1, n).contiguous().unbind(0))
            del w_all, x_all
        dist.barrier()
        if even:
            y_ref = torch.empty_like(y_ep)
            dist.scatter(y_ref, y_ref_parts, src=0)
            bad_rows = (y_ref.view(torch.int16) != y_ep.view(torch.int16)).any(dim=1).sum()
            tally = torch.stack([bad_rows.to(torch.int64),
                                 torch.tensor(y_ep.shape[0], dtype=torch.int64, device=dev)])
            dist.all_reduce(tally)
            parity = {"checked": True, "rows_compared": int(tally[1].item()),
                      "rows_differing": int(tally[0].item()),
                      "against": "the same batch through the single-GPU engine on rank 0, bitwise"}
            if parity["rows_differing"] != 0:
                raise RuntimeError(f"expert-parallel output differs from the single-GPU engine: {parity}")

    if world > 1:
        dist.barrier()
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peaks = bench.measured_peaks()
    achieved = gemm_flops_local / (gemm_ms_local * 1e-3) / 1e12
    line = {
        "metric": "useful BF16 TFLOP/s per grouped GEMM", "unit": "TFLOP/s",
        "value": total_flops / (ms_per_step * 1e-3) / 1e12,
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        # the same batch on ONE GPU in the same run, and this line's value over N times that
        "single_gpu_same_workload": single_gpu,
        "efficiency_same_workload": (total_flops / (ms_per_step * 1e-3) / 1e12
                                     / (world * single_gpu["value"]) if single_gpu else None),
        "parity_checked": bool(parity and parity["checked"]),
        "rows_compared": parity["rows_compared"] if parity else 0,
        "parity": parity,
        "p50_us": bench.percentile(step_samples, 0.5) * 1e3,
        "p99_us": bench.percentile(step_samples, 0.99) * 1e3,
        "config": {"workload": workload, "experts": spec["experts"], "top_k": top_k,
                   "tokens": tokens, "k": k, "n": n,
                   "policy": fused_policy if args.exchange == "fused" else args.policy,
                   "device_planned": bool(getattr(layer_info, "device_plan", False)),
                   "send_once": bool(getattr(layer_info, "send_once", False)),
                   "parallelism": f"ep{world}",
                   "placement": ("tile-count LPT" if parts is None else
                                 "tile-count LPT over row shards: %d of %d experts split, %d shards"
                                 % (sum(p > 1 for p in parts), len(parts), sum(parts))),
                   "exchange": args.exchange,
                   "last_step": "weighted top-k sum" if gates is not None else "rows in assignment order",
                   "pipeline_groups": groups,
                   "comm_sms": (exchange_sms_used if args.exchange == "fused"
                                else args.comm_sms if groups > 1 else 0),
                   "copy_engine_min_kb": args.copy_engine_kb if args.exchange == "fused" else None,
                   "rank0_copy_engine_bytes_per_step": copy_bytes,
                   "rank_tiles": rank_tiles, "rank0_rows": local_rows,
                   "max_rank_rows": rows_max, "mean_rank_rows": tokens * top_k / world,
                   "l2": "per-rank weights exceed the 126 MB L2; no flush between steps",
                   "note": "with more than one GPU the benchmark runs the expert-parallel "
                           "configuration; the one-GPU line of bench.py runs the "
                           "Mixtral-shaped grouped GEMM, see single_gpu_same_workload",
                   "step": ("count all-gather + push rows into the owners' packed A over "
                            "NVLink while the grouped GEMM, gated per expert group, already "
                            "computes + push result rows back"
                            if args.exchange == "fused" else
                            "count all-gather + push rows into the owners' packed A over "
                            "NVLink + grouped GEMM + pull result rows back"
                            if args.exchange == "peer" else
                            "count all-gather + pack + all-to-all dispatch + unpack + "
                            "grouped GEMM + repack + all-to-all combine + un-permute")},
        "phases_ms_max_over_ranks": phases_ms,
        "phases_note": "per-phase times come from an un-pipelined pass; the timed steps "
                       "overlap them when pipeline_groups > 1",
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": peaks["bf16_tflops"],
                     "unit": "TFLOP/s", "frac": achieved / peaks["bf16_tflops"],
                     "traffic": None, "peak_source": peaks["source"],
                     "kernel": "grouped_gemm_kernel (rank 0, GEMM phase only)",
                     "avg_launch_ms": gemm_ms_local},
        "cpu_baseline": None,
        "e2e": {"value": total_flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                "h2d_bytes_per_step": x_host.numel() * 2 * world,
                "d2h_bytes_per_step": y_host.numel() * 2 * world, "ms_per_step": e2e_ms},
        "gpu_launches": launches, "clocks": clocks,
    }
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
