"""Host-side planning interface: spec, workload plan, claim models, dispatch.

Mirrors the reference's Python planning modules name for name so that its
planner tests read the same against this package:

* ``MoESpec`` (alias ``TIRxMoESpec``), ``WorkTile``, ``MoEWorkloadPlan``,
  ``build_workload_plan``, ``static_cta_assignments``, ``chunked_claims``,
  ``hybrid_claims``  - python/blackwell_moe_tirx/config.py:20-267
* ``RoutingFeatures``, ``DispatchThresholds``, ``routing_features``,
  ``select_kernel``   - python/blackwell_moe_tirx/dispatch.py:16-114
* ``KernelDescriptor``, ``KERNEL_VERSIONS``, ``list_versions``,
  ``get_descriptor``  - python/blackwell_moe_tirx/kernels/registry.py:16-118

The arithmetic runs in the engine's C++ host library through the C interface;
this module only shapes arguments and results.
"""

from __future__ import annotations

import ctypes as C
import math
from dataclasses import dataclass, fields
from typing import Sequence

from . import _capi


@dataclass(frozen=True)
class MoESpec:
    """Shape and launch configuration (reference: ``TIRxMoESpec``).

    ``tile_n`` may be 128 or 256 here (the reference family is fixed at 128);
    ``pipe_depth`` is informational - the engine derives its stage count from
    the tile width.
    """

    experts: int = 64
    tokens: int = 4096
    n: int = 7168
    k: int = 2048
    tile_m: int = 128
    tile_n: int = 128
    tile_k: int = 64
    cta_count: int = 148
    pipe_depth: int = 2
    claim_size: int = 4
    hybrid_main_claim_size: int = 8
    hybrid_tail_tiles: int = 296
    dtype: str = "bfloat16"

    def validate(self) -> None:
        if self.experts <= 0:
            raise ValueError("experts must be positive")
        if self.tokens < 0:
            raise ValueError("tokens must be non-negative")
        if min(self.n, self.k, self.tile_m, self.tile_n, self.tile_k) <= 0:
            raise ValueError("matrix and tile dimensions must be positive")
        if self.n % 8 or self.k % 8:
            raise ValueError("n and k must be multiples of 8 (16-byte rows)")
        if self.tile_m != 128 or self.tile_n not in (128, 256) or self.tile_k != 64:
            raise ValueError(
                "the tcgen05 kernel supports a 128x128x64 or 128x256x64 CTA tile"
            )
        if self.cta_count <= 0:
            raise ValueError("cta_count must be positive")
        if self.claim_size <= 0:
            raise ValueError("claim_size must be positive")
        if self.hybrid_main_claim_size <= 0:
            raise ValueError("hybrid_main_claim_size must be positive")
        if self.hybrid_tail_tiles < 0:
            raise ValueError("hybrid_tail_tiles must be non-negative")
        if self.dtype != "bfloat16":
            raise ValueError("the engine supports BF16 inputs and output")


TIRxMoESpec = MoESpec


@dataclass(frozen=True)
class WorkTile:
    """One expert output tile; ``tile_m`` / ``tile_n`` are ELEMENT offsets."""

    expert_id: int
    tile_m: int
    tile_n: int
    valid_m: int
    valid_n: int


@dataclass(frozen=True)
class MoEWorkloadPlan:
    distribution: str
    seed: int
    tokens_per_expert: tuple[int, ...]
    tiles: tuple[WorkTile, ...]
    m_capacity: int
    logical_flops: int
    padded_flops: int
    tile_m: int = 128
    tile_n: int = 128

    @property
    def active_experts(self) -> int:
        return sum(count > 0 for count in self.tokens_per_expert)

    @property
    def useful_work_ratio(self) -> float:
        return 1.0 if self.padded_flops == 0 else self.logical_flops / self.padded_flops

    def device_worklist(self) -> list[list[int]]:
        """``[expert, m_tile_index, n_tile_index]`` triples, expert-major."""
        return [
            [t.expert_id, t.tile_m // self.tile_m, t.tile_n // self.tile_n]
            for t in self.tiles
        ]


def _counts_array(counts: Sequence[int]):
    arr = (C.c_uint32 * max(1, len(counts)))()
    for i, c in enumerate(counts):
        arr[i] = int(c)
    return arr


def generate_token_counts(
    spec: MoESpec,
    distribution: str,
    *,
    seed: int = 2026,
    zipf_alpha: float = 1.2,
    heavy_fraction: float = 0.1,
    heavy_share: float = 0.8,
    inactive_fraction: float = 0.5,
) -> tuple[int, ...]:
    """Routed rows per expert from the engine's C++ workload generator."""
    spec.validate()
    if distribution not in _capi.DISTRIBUTIONS:
        raise ValueError(f"unsupported distribution: {distribution}")
    cfg = _capi.WorkloadConfig(
        experts=spec.experts,
        distribution=_capi.DISTRIBUTIONS[distribution],
        total_tokens=spec.tokens,
        seed=seed,
        zipf_alpha=zipf_alpha,
        heavy_hitter_fraction=heavy_fraction,
        heavy_hitter_token_share=heavy_share,
        inactive_expert_fraction=inactive_fraction,
    )
    out = (C.c_uint32 * spec.experts)()
    rc = _capi.load().bmoe_generate_workload(C.byref(cfg), out)
    if rc != _capi.OK:
        raise ValueError("invalid workload configuration")
    return tuple(int(x) for x in out)


def host_tiles(
    counts: Sequence[int],
    n: int,
    tile_m: int = 128,
    tile_n: int = 128,
    *,
    order: int = _capi.ORDER_EXPERT,
    raster: int = _capi.RASTER_N_FASTEST,
):
    """Tile records (ctypes array of ``Tile``) from the host scheduler model."""
    lib = _capi.load()
    arr = _counts_array(counts)
    total = lib.bmoe_host_tile_count(arr, len(counts), n, tile_m, tile_n)
    if total == 2**64 - 1:
        raise ValueError("tile dimensions must be positive")
    tiles = (_capi.Tile * max(1, total))()
    written = C.c_uint64(0)
    rc = lib.bmoe_host_build_tiles(
        arr, len(counts), n, tile_m, tile_n, order, raster, tiles, total, C.byref(written)
    )
    if rc != _capi.OK:
        raise ValueError("invalid worklist request")
    return tiles, int(written.value)


def build_workload_plan(
    spec: MoESpec,
    distribution: str = "uniform",
    *,
    seed: int = 2026,
    token_counts: Sequence[int] | None = None,
) -> MoEWorkloadPlan:
    """Active-expert-compacted, expert-major tile work list."""
    spec.validate()
    counts = (
        generate_token_counts(spec, distribution, seed=seed)
        if token_counts is None
        else tuple(int(c) for c in token_counts)
    )
    if len(counts) != spec.experts:
        raise ValueError("token_counts length must equal experts")
    if any(c < 0 for c in counts):
        raise ValueError("token counts must be non-negative")
    if sum(counts) != spec.tokens:
        raise ValueError("token counts must sum to spec.tokens")

    records, total = host_tiles(counts, spec.n, spec.tile_m, spec.tile_n)
    tiles = tuple(
        WorkTile(
            expert_id=records[i].expert_id,
            tile_m=records[i].tile_m * spec.tile_m,
            tile_n=records[i].tile_n * spec.tile_n,
            valid_m=records[i].valid_m,
            valid_n=records[i].valid_n,
        )
        for i in range(total)
    )
    max_m = max(counts, default=0)
    m_capacity = max(spec.tile_m, math.ceil(max_m / spec.tile_m) * spec.tile_m)
    return MoEWorkloadPlan(
        distribution=distribution,
        seed=seed,
        tokens_per_expert=counts,
        tiles=tiles,
        m_capacity=m_capacity,
        logical_flops=2 * sum(counts) * spec.n * spec.k,
        padded_flops=len(tiles) * 2 * spec.tile_m * spec.tile_n * spec.k,
        tile_m=spec.tile_m,
        tile_n=spec.tile_n,
    )


def static_cta_assignments(tile_count: int, cta_count: int) -> tuple[tuple[int, ...], ...]:
    """Tiles each CTA visits under the static grid stride."""
    if tile_count < 0:
        raise ValueError("tile_count must be non-negative")
    if cta_count <= 0:
        raise ValueError("cta_count must be positive")
    return tuple(tuple(range(c, tile_count, cta_count)) for c in range(cta_count))


def chunked_claims(tile_count: int, claim_size: int) -> tuple[tuple[int, ...], ...]:
    """Contiguous batches handed out by a monotonic atomic queue."""
    if tile_count < 0:
        raise ValueError("tile_count must be non-negative")
    if claim_size <= 0:
        raise ValueError("claim_size must be positive")
    return tuple(
        tuple(range(b, min(b + claim_size, tile_count)))
        for b in range(0, tile_count, claim_size)
    )


def hybrid_claims(
    tile_count: int, main_claim_size: int, tail_tiles: int
) -> tuple[tuple[int, ...], ...]:
    """Coarse chunks first, then one tile per claim for the last ``tail_tiles``."""
    if tile_count < 0:
        raise ValueError("tile_count must be non-negative")
    if main_claim_size <= 0:
        raise ValueError("main_claim_size must be positive")
    if tail_tiles < 0:
        raise ValueError("tail_tiles must be non-negative")
    tail_begin = tile_count - min(tile_count, tail_tiles)
    main = chunked_claims(tail_begin, main_claim_size)
    return main + tuple((t,) for t in range(tail_begin, tile_count))


# --------------------------------------------------------------- dispatch --


@dataclass(frozen=True)
class RoutingFeatures:
    mean_m: float
    cv_m: float
    max_over_mean_m: float
    inactive_expert_ratio: float
    small_m_expert_ratio: float
    expert_tile_cv: float
    max_expert_tiles_over_mean: float
    active_tiles: int
    tiles_per_cta: float
    useful_work_ratio: float


@dataclass(frozen=True)
class DispatchThresholds:
    nonpersistent_tiles_per_cta: float = 1.0
    static_cv_m: float = 0.25
    dynamic_min_tiles_per_cta: float = 2.0
    chunked_min_tiles_per_cta: float = 4.0
    high_skew_cv_m: float = 1.0
    sparse_expert_ratio: float = 0.5


def _features_struct(spec: MoESpec, plan: MoEWorkloadPlan) -> _capi.RoutingFeatures:
    out = _capi.RoutingFeatures()
    counts = plan.tokens_per_expert
    rc = _capi.load().bmoe_routing_features_compute(
        _counts_array(counts), len(counts), spec.n, spec.tile_m, spec.tile_n,
        spec.cta_count, C.byref(out),
    )
    if rc != _capi.OK:
        raise ValueError("invalid routing-feature request")
    return out


def routing_features(spec: MoESpec, plan: MoEWorkloadPlan) -> RoutingFeatures:
    raw = _features_struct(spec, plan)
    return RoutingFeatures(**{f.name: getattr(raw, f.name) for f in fields(RoutingFeatures)})


def select_kernel(
    spec: MoESpec,
    plan: MoEWorkloadPlan,
    thresholds: DispatchThresholds = DispatchThresholds(),
) -> str:
    """Launch variant chosen by the threshold rule (never ``v5_clc``)."""
    raw = _features_struct(spec, plan)
    th = (C.c_double * 6)(*(getattr(thresholds, f.name) for f in fields(DispatchThresholds)))
    variant = C.c_uint32(0)
    rc = _capi.load().bmoe_select_variant(C.byref(raw), th, C.byref(variant))
    if rc != _capi.OK:
        raise ValueError("dispatch failed")
    return _capi.VARIANT_NAMES[variant.value]


# --------------------------------------------------------------- registry --


@dataclass(frozen=True)
class KernelDescriptor:
    """Launch variant metadata; all variants are modes of one sm_100a kernel."""

    name: str
    implementation: str
    persistent: bool
    warp_specialized: bool
    acquisition: str
    scheduler: str
    requires_queue: bool = False
    requires_clc: bool = False

    def launch_ctas(self, spec: MoESpec, plan: MoEWorkloadPlan) -> int:
        if self.name in {"v0_nonpersistent", "v5_clc"}:
            return len(plan.tiles)
        return spec.cta_count

    def queue_initial_values(self, spec: MoESpec, plan: MoEWorkloadPlan) -> tuple[int, int]:
        if self.name == "v4_hybrid":
            tail = min(len(plan.tiles), spec.hybrid_tail_tiles)
            return (0, len(plan.tiles) - tail)
        return (0, 0)

    def engine_options(self, spec: MoESpec) -> dict:
        """Arguments for ``GroupedGemmPlan`` that realise this variant."""
        if self.name == "v0_nonpersistent":
            return {"scheduler": "expert_order", "cta_count": 1 << 30}
        if self.name in ("v0_5_persistent", "v1_static_ws"):
            return {"scheduler": self.scheduler, "cta_count": spec.cta_count}
        if self.name == "v2_dynamic":
            return {"scheduler": "dynamic_queue", "claim_size": 1, "cta_count": spec.cta_count}
        if self.name == "v3_chunked":
            return {"scheduler": "dynamic_queue", "claim_size": spec.claim_size,
                    "cta_count": spec.cta_count}
        if self.name == "v4_hybrid":
            return {"scheduler": "dynamic_queue", "claim_size": spec.hybrid_main_claim_size,
                    "hybrid_tail_tiles": spec.hybrid_tail_tiles, "cta_count": spec.cta_count}
        return {"scheduler": "clc"}


KERNEL_VERSIONS: dict[str, KernelDescriptor] = {
    d.name: d
    for d in (
        KernelDescriptor("v0_nonpersistent", "sm100_one_cta_per_tile", False, True,
                         "one CTA per work tile", "expert_order"),
        KernelDescriptor("v0_5_persistent", "sm100_static_persistent", True, True,
                         "static grid stride", "expert_order"),
        KernelDescriptor("v1_static_ws", "sm100_static_persistent_ws", True, True,
                         "static grid stride", "static_persistent"),
        KernelDescriptor("v2_dynamic", "sm100_dynamic_claim1_ws", True, True,
                         "global atomic queue, claim 1", "dynamic_queue", requires_queue=True),
        KernelDescriptor("v3_chunked", "sm100_chunked_dynamic_ws", True, True,
                         "global atomic queue, run-time chunk", "dynamic_queue",
                         requires_queue=True),
        KernelDescriptor("v4_hybrid", "sm100_locality_hybrid_ws", True, True,
                         "expert-major coarse chunks plus fine-grained tail",
                         "dynamic_queue", requires_queue=True),
        KernelDescriptor("v5_clc", "sm100_clc_ws", True, True,
                         "Blackwell Cluster Launch Control", "clc", requires_clc=True),
    )
}


def list_versions() -> tuple[str, ...]:
    return tuple(KERNEL_VERSIONS)


def get_descriptor(version: str) -> KernelDescriptor:
    try:
        return KERNEL_VERSIONS[version]
    except KeyError as error:
        choices = ", ".join(KERNEL_VERSIONS)
        raise ValueError(
            f"unknown kernel version {version!r}; choose one of: {choices}"
        ) from error
