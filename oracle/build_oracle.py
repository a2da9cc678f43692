"""Build recipe for the checkers under oracle/ (test infrastructure only).

* ``liboracle.so``            - gcc build of bmoe_oracle.c (the CPU restatement).
* ``_ref/libref_sched.so``    - the reference's own workload.cpp / scheduler.cpp,
  compiled in place from the reference checkout together with ref_shim.cpp.
  Built only where that checkout exists; the output directory is git-ignored
  and no reference source is copied.
"""

from __future__ import annotations

import os
import subprocess
from pathlib import Path

ORACLE_DIR = Path(__file__).resolve().parent
ORACLE_LIB = ORACLE_DIR / "liboracle.so"
REF_DIR = ORACLE_DIR / "_ref"
REF_LIB = REF_DIR / "libref_sched.so"
REFERENCE_ROOT = Path(os.environ.get("BMOE_REFERENCE_ROOT", "/root/reference"))


def _run(cmd: list[str]) -> None:
    proc = subprocess.run(cmd, capture_output=True, text=True, errors="replace")
    if proc.returncode != 0:
        raise RuntimeError(f"{' '.join(cmd)}\n{proc.stdout}\n{proc.stderr[-4000:]}")


def _stale(target: Path, deps: list[Path]) -> bool:
    return not target.exists() or any(d.stat().st_mtime > target.stat().st_mtime for d in deps)


def build_oracle() -> Path:
    src = ORACLE_DIR / "bmoe_oracle.c"
    if _stale(ORACLE_LIB, [src]):
        _run(["gcc", "-O3", "-std=gnu11", "-fopenmp", "-fPIC", "-shared",
              "-fvisibility=hidden", "-Wall", str(src), "-lm", "-o", str(ORACLE_LIB)])
    return ORACLE_LIB


def reference_available() -> bool:
    return (REFERENCE_ROOT / "src" / "scheduler" / "scheduler.cpp").exists()


def build_reference() -> Path | None:
    """Compile the reference's host scheduler where its checkout is present."""
    if not reference_available():
        return REF_LIB if REF_LIB.exists() else None
    shim = ORACLE_DIR / "ref_shim.cpp"
    srcs = [REFERENCE_ROOT / "src" / "workload" / "workload.cpp",
            REFERENCE_ROOT / "src" / "scheduler" / "scheduler.cpp"]
    if _stale(REF_LIB, [shim, *srcs]):
        REF_DIR.mkdir(exist_ok=True)
        _run(["g++", "-O2", "-std=c++17", "-fPIC", "-shared",
              f"-I{REFERENCE_ROOT / 'include'}", str(shim), *map(str, srcs),
              "-o", str(REF_LIB)])
    return REF_LIB


HARNESS_DIR = REF_DIR / "bin"
# The reference's own GPU harness programs. They are compiled UNMODIFIED from the
# reference checkout, but against THIS repository's headers and engine library:
# running them on a B200 is the drop-in check for the GPU entry points.
HARNESS_SOURCES = {
    "ref_grouped_gemm_benchmark": "baselines/cutlass/benchmark.cu",
    "ref_scheduler_gpu_benchmark": "benchmarks/scheduler_gpu_benchmark.cu",
    "ref_test_scheduler_probe": "tests/test_scheduler_probe.cu",
    "ref_sm100_dense_benchmark": "benchmarks/sm100_dense_benchmark.cu",
    "ref_sm100_2sm_benchmark": "benchmarks/sm100_2sm_benchmark.cu",
    "ref_direct_cute_benchmark": "benchmarks/direct_cute_benchmark.cu",
}


def build_reference_harness() -> list[Path]:
    """nvcc-compile the reference's GPU harness against include/ + libbmoe_b200.so."""
    built = []
    if not reference_available():
        return sorted(HARNESS_DIR.glob("ref_*")) if HARNESS_DIR.exists() else built
    repo = ORACLE_DIR.parent
    lib_dir = repo / "blackwell-moe-kernel-scheduler_b200" / "lib"
    lib = lib_dir / "libbmoe_b200.so"
    if not lib.exists():
        return built
    HARNESS_DIR.mkdir(parents=True, exist_ok=True)
    for name, rel in HARNESS_SOURCES.items():
        src = REFERENCE_ROOT / rel
        out = HARNESS_DIR / name
        if _stale(out, [src, lib]):
            _run(["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-O2", "-std=c++17",
                  f"-I{repo / 'include'}", "-DBLACKWELL_MOE_CUTLASS_REVISION=\"none\"",
                  str(src), f"-L{lib_dir}", "-lbmoe_b200", "-Xlinker", "-rpath", "-Xlinker",
                  "$ORIGIN/../../../blackwell-moe-kernel-scheduler_b200/lib", "-o", str(out)])
        built.append(out)
    return built


def cutlass_include_dirs() -> list[Path]:
    """CUTLASS / CuTe header trees that happen to ship inside installed Python packages
    (the reference pins CUTLASS v4.6.0 and fetches it from the network,
    cmake/Dependencies.cmake:6-13; the copy found here may be another 4.x)."""
    import site

    for base in site.getsitepackages():
        root = Path(base) / "flashinfer" / "data" / "cutlass"
        if (root / "include" / "cutlass" / "cutlass.h").exists():
            return [root / "include", root / "tools" / "util" / "include"]
    return []


# The reference's OWN sm_100a dense kernel (CUTLASS 1-SM collective, cluster 1x1x1,
# src/kernels/sm100_dense_gemm.cu) with its own benchmark and known-answer test,
# compiled unmodified against the REFERENCE's headers: the comparison arm of the dense
# M-sweep. The 2-SM collective is left out on purpose (it relies on TMA multicast
# inside CUTLASS, include/blackwell_moe/kernels/sm100_2sm_gemm.cuh:9-12).
NATIVE_DENSE = {
    "ref_native_sm100_dense_benchmark": "benchmarks/sm100_dense_benchmark.cu",
    "ref_native_sm100_dense_test": "tests/test_sm100_dense_correctness.cu",
}


def build_reference_native_dense() -> list[Path]:
    """nvcc-compile the reference's CUTLASS dense kernel + its benchmark / test.
    Returns the programs present afterwards; raises with the compiler's output if the
    headers found do not compile it."""
    if not reference_available():
        return sorted(HARNESS_DIR.glob("ref_native_*")) if HARNESS_DIR.exists() else []
    includes = cutlass_include_dirs()
    if not includes:
        return []
    HARNESS_DIR.mkdir(parents=True, exist_ok=True)
    kernel_src = REFERENCE_ROOT / "src" / "kernels" / "sm100_dense_gemm.cu"
    shim = ORACLE_DIR / "ref_status_shim.cpp"
    flags = ["-gencode", "arch=compute_100a,code=sm_100a", "-O2", "-std=c++17",
             "--expt-relaxed-constexpr", "-diag-suppress", "20012",
             f"-I{REFERENCE_ROOT / 'include'}", *[f"-I{d}" for d in includes],
             "-DBLACKWELL_MOE_CUTLASS_REVISION=\"4.5.0-vendored-headers\""]
    kernel_obj = REF_DIR / "ref_native_sm100_dense_gemm.o"
    if _stale(kernel_obj, [kernel_src]):
        _run(["nvcc", *flags, "-c", str(kernel_src), "-o", str(kernel_obj)])
    shim_obj = REF_DIR / "ref_status_shim.o"
    if _stale(shim_obj, [shim]):
        _run(["nvcc", *flags, "-x", "cu", "-c", str(shim), "-o", str(shim_obj)])
    built = []
    for name, rel in NATIVE_DENSE.items():
        src = REFERENCE_ROOT / rel
        out = HARNESS_DIR / name
        if _stale(out, [src, kernel_obj, shim_obj]):
            _run(["nvcc", *flags, str(src), str(shim_obj), str(kernel_obj), "-o", str(out)])
        built.append(out)
    return built


if __name__ == "__main__":
    print(build_oracle())
    print(build_reference())
    print(build_reference_harness())
    print(build_reference_native_dense())
