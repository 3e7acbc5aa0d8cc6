"""Build libds4b200.so (the CUDA kernels and their C ABI) in-tree for sm_100a.

    python -m ds4cuda_b200.build [--force] [--verbose]

nvcc cross-compiles without a GPU.  Objects and the library are written next to
this file (git-ignored); the library is the only artefact the Python side loads.
"""
from __future__ import annotations

import argparse
import concurrent.futures
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
INCLUDE = PKG.parent / "include"
LIB = PKG / "libds4b200.so"
SOURCES = ["norm.cu", "embedding.cu", "rope_fp8.cu", "glu.cu", "quant.cu", "hc.cu", "hc_pre_cluster.cu", "hc_pre_mma.cu", "hc_pre_tc.cu", "compressor.cu", "layer.cu", "noalloc.cu", "path.cu",
           "launchers.cu", "capi.cu"]
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def nvcc() -> str:
    exe = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(exe).exists():
        raise RuntimeError("nvcc not found (set NVCC=/path/to/nvcc)")
    return exe


def _stale(target: Path, deps: list[Path]) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    headers = sorted(CSRC.glob("*.cuh")) + sorted(INCLUDE.glob("*"))
    obj_dir = PKG / "build"
    obj_dir.mkdir(exist_ok=True)
    sources = [CSRC / s for s in SOURCES if (CSRC / s).exists()]
    flags = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", *ARCH]
    if verbose:
        flags += ["-Xptxas", "-v"]

    def compile_one(src: Path) -> Path:
        obj = obj_dir / (src.stem + ".o")
        if force or _stale(obj, [src, *headers]):
            cmd = [nvcc(), *flags, "-c", str(src), "-o", str(obj)]
            r = subprocess.run(cmd, capture_output=True, text=True)
            if verbose or r.returncode:
                sys.stderr.write(r.stdout + r.stderr)
            if r.returncode:
                raise RuntimeError(f"nvcc failed on {src.name}")
        return obj

    with concurrent.futures.ThreadPoolExecutor(max_workers=8) as ex:
        objs = list(ex.map(compile_one, sources))
    if force or _stale(LIB, objs):
        cmd = [nvcc(), "-shared", *ARCH, "-o", str(LIB), *map(str, objs)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("link failed")
    return LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    print(build(a.force, a.verbose))
