"""In-tree build of the engine's shared library for sm_100a.

``build_library()`` compiles every source under ``csrc/`` with nvcc
(``-gencode arch=compute_100a,code=sm_100a``; cross-compiles without a GPU) and
links ``lib/libbmoe_b200.so`` next to this file. Objects are rebuilt only when a
source or header is newer than the object.
"""

from __future__ import annotations

import os
import shutil
import subprocess
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
REPO_ROOT = PKG_DIR.parent
CSRC = PKG_DIR / "csrc"
LIB_DIR = PKG_DIR / "lib"
OBJ_DIR = PKG_DIR / "build"
LIB_PATH = LIB_DIR / "libbmoe_b200.so"
# The same sources with -DBMOE_CHECKS: every tile record is bounds-checked on the device
# before it is used (a failure is a reported status, never a trap). Loaded instead of the
# plain library when the environment has BMOE_CHECKS=1.
CHECKS_LIB_PATH = LIB_DIR / "libbmoe_b200_checks.so"
CHECKS_OBJ_DIR = PKG_DIR / "build_checks"

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON_FLAGS = [
    "-O3",
    "-std=c++17",
    "-lineinfo",
    "-Xcompiler",
    "-fPIC",
    "-Xcompiler",
    "-Wall",
    f"-I{REPO_ROOT / 'include'}",
    f"-I{CSRC / 'cuda'}",
]


def _nvcc() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(found):
        raise RuntimeError("nvcc not found; the engine has no non-CUDA build")
    return found


def sources() -> list[Path]:
    return sorted((CSRC / "host").glob("*.cpp")) + sorted((CSRC / "cuda").glob("*.cu"))


def _headers() -> list[Path]:
    return (
        list((REPO_ROOT / "include").rglob("*.h"))
        + list((REPO_ROOT / "include").rglob("*.hpp"))
        + list((REPO_ROOT / "include").rglob("*.cuh"))
        + list((CSRC / "cuda").glob("*.cuh"))
    )


def _compile_one(src: Path, newest_header: float, verbose: bool, checks: bool = False) -> Path:
    obj = (CHECKS_OBJ_DIR if checks else OBJ_DIR) / (src.stem + ".o")
    if obj.exists() and obj.stat().st_mtime >= max(src.stat().st_mtime, newest_header):
        return obj
    cmd = [_nvcc(), *ARCH_FLAGS, *COMMON_FLAGS]
    if checks:
        cmd.append("-DBMOE_CHECKS")
    if src.suffix == ".cu" and verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += ["-c", str(src), "-o", str(obj)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{proc.stdout}\n{proc.stderr}")
    if verbose and proc.stderr.strip():
        print(proc.stderr)
    return obj


def build_library(force: bool = False, verbose: bool = False, checks: bool = False) -> Path:
    """Compile and link ``libbmoe_b200.so`` (``checks``: the bounds-checked
    ``libbmoe_b200_checks.so``); returns its path."""
    lib_path = CHECKS_LIB_PATH if checks else LIB_PATH
    obj_dir = CHECKS_OBJ_DIR if checks else OBJ_DIR
    LIB_DIR.mkdir(exist_ok=True)
    obj_dir.mkdir(exist_ok=True)
    if force:
        for old in obj_dir.glob("*.o"):
            old.unlink()
    srcs = sources()
    newest_header = max(h.stat().st_mtime for h in _headers())
    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as pool:
        objs = list(pool.map(lambda s: _compile_one(s, newest_header, verbose, checks), srcs))
    if lib_path.exists() and all(lib_path.stat().st_mtime >= o.stat().st_mtime for o in objs):
        return lib_path
    # link beside the target, then rename: a reader never sees a half-written library
    staged = lib_path.with_suffix(".so.tmp")
    cmd = [_nvcc(), *ARCH_FLAGS, "-shared", "-o", str(staged), *map(str, objs)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"link failed:\n{proc.stdout}\n{proc.stderr}")
    os.replace(staged, lib_path)
    return lib_path


if __name__ == "__main__":
    import sys

    path = build_library(force="--force" in sys.argv, verbose="-v" in sys.argv,
                         checks="--checks" in sys.argv)
    print(path)
