"""Build libcacheir_b200.so in-tree with nvcc for sm_100a.

Usage: python -m cacheir_b200.build [--force] [--verbose]

The library is a plain C-ABI shared object (no torch, no pybind): every .cu
under csrc/ is compiled to an object with -gencode arch=compute_100a,code=sm_100a
and linked with the static CUDA runtime. Objects are rebuilt only when their
source or a header is newer.
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
INCLUDE = PKG_DIR.parent / "include"
BUILD_DIR = PKG_DIR / "build"
LIB_PATH = PKG_DIR / "lib" / "libcacheir_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def find_nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(nvcc).exists():
        raise RuntimeError("nvcc not found; cacheir_b200 needs the CUDA toolkit to build its kernels")
    return nvcc


def _stale(target: Path, deps: list[Path]) -> bool:
    if not target.exists():
        return True
    mtime = target.stat().st_mtime
    return any(dep.stat().st_mtime > mtime for dep in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    nvcc = find_nvcc()
    BUILD_DIR.mkdir(parents=True, exist_ok=True)
    LIB_PATH.parent.mkdir(parents=True, exist_ok=True)
    sources = sorted(CSRC.glob("*.cu"))
    headers = sorted(CSRC.glob("*.cuh")) + sorted(INCLUDE.glob("*.h")) + [Path(__file__)]
    extra = ["-Xptxas", "-v"] if verbose else []

    def compile_one(src: Path) -> Path:
        obj = BUILD_DIR / (src.stem + ".o")
        if force or _stale(obj, [src] + headers):
            cmd = [nvcc, *NVCC_FLAGS, *extra, "-I", str(INCLUDE), "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
            proc = subprocess.run(cmd, capture_output=True, text=True)
            if verbose or proc.returncode != 0:
                sys.stderr.write(proc.stdout + proc.stderr)
            if proc.returncode != 0:
                raise RuntimeError(f"nvcc failed on {src.name}")
        return obj

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        objects = list(pool.map(compile_one, sources))

    if force or _stale(LIB_PATH, objects):
        cmd = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-cudart", "static",
               "-o", str(LIB_PATH), *map(str, objects)]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            sys.stderr.write(proc.stdout + proc.stderr)
            raise RuntimeError("linking libcacheir_b200.so failed")
    return LIB_PATH


if __name__ == "__main__":
    parser = argparse.ArgumentParser(description=__doc__)
    parser.add_argument("--force", action="store_true")
    parser.add_argument("--verbose", action="store_true", help="print ptxas register/smem usage")
    args = parser.parse_args()
    print(build(force=args.force, verbose=args.verbose))
