"""The reference's OWN GPU programs (compiled unmodified from its checkout, against
this repository's headers and library, into oracle/_ref/bin by
oracle/build_oracle.py) run on the engine: its scheduler-probe test, its
grouped-GEMM benchmark, its probe benchmark and its three dense benchmarks.
Skipped where the binaries were not built (no reference checkout at build time)."""

import subprocess
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
BIN = Path(__file__).resolve().parent.parent / "oracle" / "_ref" / "bin"


def run(name, *args):
    exe = BIN / name
    if not exe.exists():
        pytest.skip(f"{exe} not built")
    proc = subprocess.run([str(exe), *args], capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stdout + proc.stderr
    return proc.stdout


def test_reference_probe_test_passes(engine):
    assert "GPU scheduler probe correctness passed" in run("ref_test_scheduler_probe")


def test_reference_grouped_benchmark_runs(engine):
    out = run("ref_grouped_gemm_benchmark", "--distribution=zipf", "--experts=64", "--tokens=4096",
              "--n=7168", "--k=2048", "--warmup=5", "--iterations=20", "--csv")
    header, row = out.strip().splitlines()[-2:]
    cols = dict(zip(header.split(","), row.split(",")))
    assert int(cols["active_experts"]) > 0 and float(cols["tflops"]) > 50.0
    assert int(cols["threadblocks"]) > 0


def test_reference_probe_benchmark_runs(engine):
    for scheduler in ("static", "dynamic"):
        out = run("ref_scheduler_gpu_benchmark", f"--scheduler={scheduler}", "--iterations=5",
                  "--warmup=2")
        assert out.strip()


@pytest.mark.parametrize("name", ["ref_sm100_dense_benchmark", "ref_sm100_2sm_benchmark",
                                  "ref_direct_cute_benchmark"])
def test_reference_dense_benchmarks_run(engine, name):
    out = run(name, "--m=1024", "--n=1024", "--k=512", "--warmup=3", "--iterations=10")
    assert out.strip()
