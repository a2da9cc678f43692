"""B200 (sm_100a) BF16 MoE grouped-GEMM engine behind the reference's API.

Sub-modules:
  _build    nvcc build of ``lib/libbmoe_b200.so``
  _capi     ctypes binding of ``include/bmoe_b200.h``
  planner   host planning interface (spec, worklist plan, claims, dispatch)
  engine    grouped-GEMM plan, device worklist builder, scheduler probe
  runner    correctness + CUDA-event benchmark harness (reference CSV schema), cli
  ep        expert-parallel layer (torch.distributed all-to-all)
  ep_peer   expert-parallel layer over peer memory (two routing kernels)
  ep_fused  expert-parallel layer whose exchange overlaps the grouped GEMM

The directory name contains hyphens; import it through the ``bmoe_b200`` module
at the repository root.
"""

from . import _capi  # noqa: F401
from .planner import (  # noqa: F401
    DispatchThresholds,
    KERNEL_VERSIONS,
    KernelDescriptor,
    MoESpec,
    MoEWorkloadPlan,
    RoutingFeatures,
    TIRxMoESpec,
    WorkTile,
    build_workload_plan,
    chunked_claims,
    generate_token_counts,
    get_descriptor,
    host_tiles,
    hybrid_claims,
    list_versions,
    routing_features,
    select_kernel,
    static_cta_assignments,
)
from .runner import BenchmarkResult, load_token_counts, run_benchmark  # noqa: F401
from .engine import (  # noqa: F401
    GroupedGemmPlan,
    TILE_DTYPE,
    build_worklist_on_device,
    grouped_gemm,
    launch_scheduler_probe,
    read_worklist_arrays,
    tiles_to_numpy,
    worklist_layout,
)

__all__ = [name for name in dir() if not name.startswith("_")]
