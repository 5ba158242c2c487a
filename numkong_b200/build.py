"""Builds libnumkong_b200.so in-tree with nvcc for sm_100a.

    python numkong_b200/build.py            # incremental (run as a script: importing the package needs the library)
    python numkong_b200/build.py --force    # rebuild everything

Every .cu file under csrc/ is compiled to an object (in parallel) and linked into one shared
library next to this file. The CUDA runtime is linked statically, so the library depends only
on the driver (libcuda.so.1) at run time.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
BUILD = HERE / "_build"
LIB = HERE / "libnumkong_b200.so"

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
CFLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC,-fvisibility=hidden", "--expt-relaxed-constexpr"]


def _newest_header_mtime() -> float:
    headers = list(CSRC.glob("*.h")) + list(CSRC.glob("*.cuh")) + list((HERE.parent / "include").glob("*.h"))
    return max((h.stat().st_mtime for h in headers), default=0.0)


def _compile(src: Path, obj: Path, verbose: bool) -> str:
    cmd = [NVCC, *ARCH, *CFLAGS, "-c", str(src), "-o", str(obj)]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{res.stdout}\n{res.stderr}")
    return res.stderr


def build(force: bool = False, verbose: bool = False) -> Path:
    BUILD.mkdir(exist_ok=True)
    sources = sorted(CSRC.glob("*.cu"))
    header_mtime = _newest_header_mtime()
    jobs = []
    for src in sources:
        obj = BUILD / (src.stem + ".o")
        stale = force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, header_mtime)
        if stale:
            jobs.append((src, obj))
    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as pool:
            for log in pool.map(lambda j: _compile(j[0], j[1], verbose), jobs):
                if verbose and log:
                    print(log)
    objs = [BUILD / (s.stem + ".o") for s in sources]
    if jobs or not LIB.exists():
        cmd = [NVCC, *ARCH, "-shared", "-o", str(LIB), *map(str, objs), "-cudart", "static", "-lpthread", "-ldl", "-lrt"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    return LIB


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv or "-v" in sys.argv)
    print(path)
