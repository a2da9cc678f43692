"""The bounds-checked build (-DBMOE_CHECKS, ``libbmoe_b200_checks.so``): the same sources with
every tile record verified on the device before it reaches the TMA, MMA and epilogue roles
(worklist index, expert id, column and row extents, packed-row range, k-block coverage,
Tensor Memory columns); a violation is a reported status, never a trap. compute-sanitizer
is not available where this runs, so this build, exact-once tile counters and the oracle
comparison stand in for it: the ragged, packed-descriptor and FP8 cases run again in a child
process that loads the checked library, and must pass unchanged."""

import os
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def test_checked_build_passes_the_ragged_cases(engine):
    import __graft_entry__  # noqa: F401  (repo root on sys.path)
    from bmoe_b200 import _build

    lib = _build.build_library(checks=True)
    assert lib.name == "libbmoe_b200_checks.so" and lib.exists()
    env = dict(os.environ, BMOE_CHECKS="1")
    probe = subprocess.run(
        [sys.executable, "-c",
         "import bmoe_b200; print(bmoe_b200._capi.LIB_PATH.name); bmoe_b200._capi.load()"],
        cwd=ROOT, env=env, capture_output=True, text=True, timeout=300)
    assert probe.returncode == 0, probe.stderr
    assert probe.stdout.strip() == "libbmoe_b200_checks.so"
    proc = subprocess.run(
        [sys.executable, "-m", "pytest", "-x", "-q", "-m", "gpu",
         "tests/test_gpu_gemm.py", "tests/test_gpu_fp8.py", "-k",
         "ragged or single_descriptor or reusable or fp32_output"],
        cwd=ROOT, env=env, capture_output=True, text=True, timeout=1500)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-2000:]
    assert " passed" in proc.stdout and "failed" not in proc.stdout
