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
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"{' '.join(cmd)}\n{proc.stdout}\n{proc.stderr}")


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


if __name__ == "__main__":
    print(build_oracle())
    print(build_reference())
