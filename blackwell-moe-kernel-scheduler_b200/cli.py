"""Command line of the harness: ``python bmoe_b200.py [options]``.

Same options and output as the reference's ``python -m blackwell_moe_tirx.cli``
(python/blackwell_moe_tirx/cli.py:14-118), plus ``--workload-file`` for a routing
file written by the reference's ``python/generate_workloads.py``. ``--dump-cuda``
is refused: nothing is generated at run time.
"""

from __future__ import annotations

import argparse
from pathlib import Path

from .planner import MoESpec, build_workload_plan, list_versions, routing_features, select_kernel
from .runner import BenchmarkResult, load_token_counts, run_benchmark


def build_parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(
        description="Check and benchmark a launch variant of the sm_100a grouped-GEMM kernel")
    parser.add_argument("--kernel", choices=("auto", *list_versions()), default="v1_static_ws")
    parser.add_argument("--distribution", choices=("uniform", "heavy_hitter", "sparse", "zipf", "heavy_sparse"),
                        default="uniform")
    parser.add_argument("--experts", type=int, default=64)
    parser.add_argument("--tokens", type=int, default=4096)
    parser.add_argument("--n", type=int, default=7168)
    parser.add_argument("--k", type=int, default=2048)
    parser.add_argument("--seed", type=int, default=2026)
    parser.add_argument("--ctas", type=int, default=148)
    parser.add_argument("--pipe-depth", type=int, default=2)
    parser.add_argument("--claim-size", type=int, default=4)
    parser.add_argument("--hybrid-main-claim-size", type=int, default=8)
    parser.add_argument("--hybrid-tail-tiles", type=int, default=296,
                        help="tiles reserved for claim-1 acquisition at the end of v4_hybrid")
    parser.add_argument("--warmup", type=int, default=20)
    parser.add_argument("--iterations", type=int, default=200)
    parser.add_argument("--correctness-only", action="store_true")
    parser.add_argument("--smoke", action="store_true",
                        help="small first-run shape (4 experts, 128 tokens, 256 x 256)")
    parser.add_argument("--dump-cuda", type=Path)
    parser.add_argument("--csv", action="store_true")
    parser.add_argument("--workload-file", type=Path,
                        help="tokens per expert from generate_workloads.py (JSON or CSV); "
                             "overrides --distribution / --experts / --tokens / --seed")
    return parser


def main(argv=None) -> None:
    args = build_parser().parse_args(argv)
    if args.smoke:
        args.experts, args.tokens, args.n, args.k = 4, 128, 256, 256
        args.warmup = min(args.warmup, 5)
        args.iterations = min(args.iterations, 20)
    counts = None
    if args.workload_file is not None:
        counts, args.distribution, args.seed = load_token_counts(args.workload_file)
        args.experts, args.tokens = len(counts), sum(counts)

    spec = MoESpec(experts=args.experts, tokens=args.tokens, n=args.n, k=args.k,
                   cta_count=args.ctas, pipe_depth=args.pipe_depth, claim_size=args.claim_size,
                   hybrid_main_claim_size=args.hybrid_main_claim_size,
                   hybrid_tail_tiles=args.hybrid_tail_tiles)
    if counts is None:
        plan = build_workload_plan(spec, args.distribution, seed=args.seed)
    else:
        plan = build_workload_plan(spec, args.distribution, seed=args.seed, token_counts=counts)
    chosen = select_kernel(spec, plan) if args.kernel == "auto" else args.kernel
    result = run_benchmark(spec, plan, version=chosen, warmup=args.warmup,
                           iterations=args.iterations, correctness_only=args.correctness_only,
                           dump_cuda=args.dump_cuda)
    if args.csv:
        print(BenchmarkResult.csv_header())
        print(result.csv_row())
        return
    print(f"BF16 MoE grouped GEMM correctness passed on {result.device}: kernel={chosen}, "
          f"active_experts={result.active_experts}, tiles={result.tiles}, "
          f"max_abs_error={result.max_abs_error:.6g}, max_rel_error={result.max_rel_error:.6g}")
    if not args.correctness_only:
        print(f"median={result.median_ms:.6f} ms, p95={result.p95_ms:.6f} ms, "
              f"effective={result.effective_tflops:.3f} TFLOP/s, "
              f"useful_work_ratio={result.useful_work_ratio:.3%}")
    if args.kernel == "auto":
        features = routing_features(spec, plan)
        print("bootstrap dispatch features: "
              f"cv_m={features.cv_m:.3f}, inactive_experts={features.inactive_expert_ratio:.3%}, "
              f"tiles_per_cta={features.tiles_per_cta:.3f}")


if __name__ == "__main__":
    main()
