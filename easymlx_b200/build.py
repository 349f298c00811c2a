"""Build the CUDA library in-tree: ``python -m easymlx_b200.build``.

Compiles every ``csrc/*.cu`` for sm_100a with nvcc and links
``easymlx_b200/lib/libeasymlx_b200.so`` (static CUDA runtime, no torch types,
plain C ABI declared in ``include/easymlx_b200.h``).  Objects are rebuilt only
when a source or header is newer.
"""

from __future__ import annotations

import glob
import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
LIB_DIR = os.path.join(PKG, "lib")
LIB = os.path.join(LIB_DIR, "libeasymlx_b200.so")
INCLUDE = os.path.join(os.path.dirname(PKG), "include")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; the CUDA library cannot be built")
    return exe


def build(verbose: bool = False, force: bool = False, ptxas_info: bool = False) -> str:
    os.makedirs(LIB_DIR, exist_ok=True)
    sources = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    headers = glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(INCLUDE, "*.h"))
    newest_header = max(os.path.getmtime(h) for h in headers)
    objects, jobs = [], []
    for src in sources:
        obj = os.path.join(LIB_DIR, os.path.basename(src)[:-3] + ".o")
        objects.append(obj)
        stale = force or not os.path.exists(obj) or os.path.getmtime(obj) < max(os.path.getmtime(src), newest_header)
        if not stale:
            continue
        cmd = [_nvcc(), *NVCC_FLAGS, *os.environ.get("EMLX_NVCC_EXTRA", "").split(), "-I", INCLUDE, "-c", src, "-o", obj]
        if ptxas_info:
            cmd += ["-Xptxas", "-v"]
        jobs.append(cmd)
    rebuilt = bool(jobs)

    def compile_one(cmd):
        if verbose:
            print(" ".join(cmd), flush=True)
        subprocess.run(cmd, check=True)

    # the files are independent; the largest one (the tiled attention kernels, two variants of 36 instances) sets the time
    workers = max(1, min(len(jobs), os.cpu_count() or 1, 8))
    if jobs:
        from concurrent.futures import ThreadPoolExecutor
        with ThreadPoolExecutor(workers) as pool:
            list(pool.map(compile_one, jobs))
    if rebuilt or not os.path.exists(LIB):
        cmd = [_nvcc(), "-shared", "-o", LIB, *objects]
        if verbose:
            print(" ".join(cmd), flush=True)
        subprocess.run(cmd, check=True)
    return LIB


if __name__ == "__main__":
    print(build(verbose=True, force="--force" in sys.argv, ptxas_info="--ptxas" in sys.argv))
