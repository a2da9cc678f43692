"""Drop-in check: the reference's own host programs compile against this
repository's include/blackwell_moe headers, link against the engine library and
pass. Runs only where the reference checkout is present; nothing is copied."""

import os
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
REFERENCE = Path(os.environ.get("BMOE_REFERENCE_ROOT", "/root/reference"))
LIB_DIR = ROOT / "blackwell-moe-kernel-scheduler_b200" / "lib"

pytestmark = pytest.mark.skipif(not (REFERENCE / "tests" / "test_scheduler.cpp").exists(),
                                reason="reference checkout not present")


def build(src: Path, out: Path) -> None:
    cmd = ["g++", "-std=c++17", "-O1", f"-I{ROOT / 'include'}", str(src), f"-L{LIB_DIR}",
           "-lbmoe_b200", f"-Wl,-rpath,{LIB_DIR}", "-o", str(out)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    assert proc.returncode == 0, proc.stderr


@pytest.mark.parametrize("name", ["test_workload", "test_scheduler"])
def test_reference_unit_tests_pass_against_engine_library(engine, tmp_path, name):
    exe = tmp_path / name
    build(REFERENCE / "tests" / f"{name}.cpp", exe)
    proc = subprocess.run([str(exe)], capture_output=True, text=True)
    assert proc.returncode == 0, proc.stdout + proc.stderr
    assert "passed" in proc.stdout


def test_reference_cli_runs_against_engine_library(engine, tmp_path):
    exe = tmp_path / "moe_workload_bench"
    build(REFERENCE / "benchmarks" / "benchmark_main.cpp", exe)
    for sched in ("expert_order", "static_persistent", "dynamic_queue", "compacted", "auto"):
        proc = subprocess.run([str(exe), "--distribution=zipf", "--experts=8", "--tokens=8192",
                               "--n=14336", "--k=4096", f"--scheduler={sched}", "--ctas=148",
                               "--csv"], capture_output=True, text=True)
        assert proc.returncode == 0, proc.stderr
        header, row = proc.stdout.strip().splitlines()[:2]
        assert "tail_ratio" in header and sched in row
