"""Builds the REFERENCE project's own CUDA kernels for this path as an
on-device checker: ``oracle/_ref/libkernel_set_ref.so``. TEST INFRASTRUCTURE.

The sources are compiled where they lie in a checkout of the reference project
(environment variable ``KS_REFERENCE_ROOT``, else a checkout named ``reference`` beside this
repository); nothing is copied. The result
is git-ignored. When the checkout is absent (a machine that only received the
prebuilt file) the function reports that and returns ``None``.

Only the seven translation units of the quantized-GEMM path are compiled, with
nvcc directly (the reference's CMake build is not used):
  kernels/src/common/runtime.cu, gemm/gemm_fp8_blockwise.cu, gemm/gemm_w4a16.cu,
  quant/quant_fp8_group.cu, quant/dequant_int4.cu, quant/repack_int4.cu,
  moe/moe_grouped_gemm.cu
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
OUT = os.path.join(OUT_DIR, "libkernel_set_ref.so")
SOURCES = [
    "kernels/src/common/runtime.cu",
    "kernels/src/gemm/gemm_fp8_blockwise.cu",
    "kernels/src/gemm/gemm_w4a16.cu",
    "kernels/src/quant/quant_fp8_group.cu",
    "kernels/src/quant/dequant_int4.cu",
    "kernels/src/quant/repack_int4.cu",
    "kernels/src/moe/moe_grouped_gemm.cu",
]


def build_ref(verbose: bool = False):
    root = os.environ.get("KS_REFERENCE_ROOT")
    if not root:
        # a checkout named `reference` beside this repository, if there is one
        beside = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference")
        root = beside if os.path.isdir(beside) else ""
    if not os.path.isdir(os.path.join(root, "kernels", "src")):
        return OUT if os.path.exists(OUT) else None
    srcs = [os.path.join(root, s) for s in SOURCES]
    if os.path.exists(OUT) and all(os.path.getmtime(OUT) >= os.path.getmtime(s) for s in srcs):
        return OUT
    os.makedirs(OUT_DIR, exist_ok=True)
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    cmd = [nvcc, "-shared", "-o", OUT, "-O3", "-std=c++17", "-lineinfo",
           "-gencode", "arch=compute_100,code=sm_100",
           "-Xcompiler", "-fPIC,-fvisibility=hidden", "-DKERNEL_SET_BUILD", "-DKS_ENABLE_CUDA",
           "-I", os.path.join(root, "include"), "-I", os.path.join(root, "kernels", "src"), *srcs]
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("reference kernels did not compile:\n" + r.stdout + r.stderr)
    return OUT


if __name__ == "__main__":
    print(build_ref(verbose="-v" in sys.argv))
