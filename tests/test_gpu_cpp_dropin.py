"""Runs the compiled C++ drop-in program (tests/cpp/dropin_gpu_test.cu): the
reference's GPU known-answer tests against the C++ classes of this engine
(grouped plan with all six policies, 1-CTA and CTA-pair dense plans, the FP32
one-shot launcher, the scheduler probe)."""

import subprocess
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def test_cpp_dropin_program(engine):
    import __graft_entry__ as entry

    exe = entry.build_cpp_tests()
    proc = subprocess.run([str(exe)], capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0, proc.stdout + proc.stderr
    assert "drop-in GPU tests passed" in proc.stdout
