"""In-tree build of ``libkernel_set.so`` for sm_100a with plain nvcc.

``python -m kernel_set_b200.build`` compiles every ``csrc/*.cu`` (objects are
rebuilt only when a source or header is newer) and links
``kernel_set_b200/lib/libkernel_set.so``, the drop-in for the reference
project's library of the same name (built there by CMake,
``CMakeLists.txt:25-69``: hidden visibility, ``-lineinfo``, no fast-math).

nvcc cross-compiles without a GPU, so this also runs on a CPU-only machine.
"""
from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "_obj")
LIB_DIR = os.path.join(HERE, "lib")
LIB = os.path.join(LIB_DIR, "libkernel_set.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden",
    "-DKERNEL_SET_BUILD",
    "-I", os.path.join(ROOT, "include"),
    "-I", CSRC,
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; the library has no CPU build")
    return exe


def _newest_header() -> float:
    newest = 0.0
    for base in (CSRC, os.path.join(ROOT, "include", "kernel_set")):
        for name in os.listdir(base):
            if name.endswith((".cuh", ".h")):
                newest = max(newest, os.path.getmtime(os.path.join(base, name)))
    return newest


def build(verbose: bool = False, force: bool = False) -> str:
    """Compile and link the library; returns its path."""
    os.makedirs(OBJ, exist_ok=True)
    os.makedirs(LIB_DIR, exist_ok=True)
    nvcc = _nvcc()
    header_time = _newest_header()
    sources = sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))
    jobs = []
    objects = []
    for src in sources:
        s = os.path.join(CSRC, src)
        o = os.path.join(OBJ, src[:-3] + ".o")
        objects.append(o)
        stale = force or not os.path.exists(o) or os.path.getmtime(o) < max(os.path.getmtime(s), header_time)
        if stale:
            jobs.append([nvcc, *NVCC_FLAGS, "-c", s, "-o", o])

    def run(cmd):
        if verbose:
            print(" ".join(cmd), flush=True)
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed:\n" + " ".join(cmd) + "\n" + r.stdout + r.stderr)

    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        list(pool.map(run, jobs))

    if jobs or not os.path.exists(LIB):
        run([nvcc, "-shared", "-o", LIB, *objects, "-Xcompiler", "-fvisibility=hidden",
             "-gencode", "arch=compute_100a,code=sm_100a"])
    return LIB


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force="-f" in sys.argv))
