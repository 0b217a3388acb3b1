"""Compile the CUDA sources of this package into libfm_b200.so (sm_100a only).

Usage: python flash-moe_b200/build.py [--force] [--verbose]
"""
from __future__ import annotations

import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
OBJ = HERE / "build"
LIB = HERE / "libfm_b200.so"

import os

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-Xptxas", "-v",
              *os.environ.get("FM_EXTRA_NVCC_FLAGS", "").split()]


def sources():
    return sorted(CSRC.glob("*.cu"))


def _newest_header() -> float:
    hs = list(CSRC.glob("*.h")) + list(CSRC.glob("*.cuh")) + list((HERE.parent / "include").glob("*.h"))
    return max(h.stat().st_mtime for h in hs)


def _compile(src: Path, force: bool, verbose: bool) -> Path:
    obj = OBJ / (src.stem + ".o")
    if not force and obj.exists() and obj.stat().st_mtime >= max(src.stat().st_mtime, _newest_header()):
        return obj
    r = subprocess.run(["nvcc", *NVCC_FLAGS, "-c", str(src), "-o", str(obj)], capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src.name}:\n{r.stdout}\n{r.stderr}")
    (OBJ / (src.stem + ".ptxas.txt")).write_text(r.stderr)
    if verbose:
        print(r.stderr)
    return obj


def build(force: bool = False, verbose: bool = False) -> Path:
    OBJ.mkdir(exist_ok=True)
    with ThreadPoolExecutor(8) as ex:
        objs = list(ex.map(lambda s: _compile(s, force, verbose), sources()))
    if force or not LIB.exists() or LIB.stat().st_mtime < max(o.stat().st_mtime for o in objs):
        subprocess.check_call(["nvcc", "-shared", "-o", str(LIB), *map(str, objs), "-lcudart"])
    return LIB


if __name__ == "__main__":
    print(build("--force" in sys.argv, "--verbose" in sys.argv))
