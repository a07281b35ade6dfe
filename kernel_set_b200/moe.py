"""Out-parameter wrappers of the grouped GEMMs; ``grouped_gemm`` has the
signature of ``bindings/python/kernel_set/moe.py:189-217`` of the reference
project, ``grouped_gemm_fp8_blockwise`` wraps the added block-scaled symbol."""
from __future__ import annotations

from typing import Optional

import torch

from ._lib import check, lib
from ._tensor import TensorLike, default_stream, dtype_to_ks, f32_ptr, i32_ptr, infer_dtype, ptr


def grouped_gemm(c: TensorLike, a: TensorLike, b: TensorLike, expert_offsets: TensorLike, num_experts: int,
                 total_rows: int, n: int, k: int, dtype: Optional[int] = None,
                 stream: TensorLike = None) -> TensorLike:
    """For each expert e: ``C[off_e:off_{e+1}] = A[off_e:off_{e+1}] @ B[e]``;
    ``b [num_experts, k, n]``, ``expert_offsets [num_experts+1]`` int32."""
    dt = infer_dtype(a, dtype)
    check(lib.ks_moe_grouped_gemm(ptr(c, name="c"), ptr(a, name="a"), ptr(b, name="b"),
                                  i32_ptr(expert_offsets, name="expert_offsets"), int(num_experts),
                                  int(total_rows), int(n), int(k), dt, default_stream(stream, a)),
          "ks_moe_grouped_gemm")
    return c


def grouped_gemm_fp8_blockwise(out: TensorLike, a_fp8: TensorLike, b_fp8: TensorLike, a_scale: TensorLike,
                               b_scale: TensorLike, expert_offsets: TensorLike, num_experts: int,
                               total_rows: int, n: int, k: int, block_n: int = 128, block_k: int = 128,
                               b_layout: str = "nk", fp8_dtype: Optional[int] = None,
                               out_dtype: Optional[int] = None, stream: TensorLike = None) -> TensorLike:
    """Per-expert FP8 block-scaled GEMM over rows sorted by expert.
    ``b_layout="nk"``: ``b_fp8 [E,N,K]``, ``b_scale [E, N/bn, K/bk]``;
    ``"kn"``: ``b_fp8 [E,K,N]``, ``b_scale [E, K/bk, N/bn]``."""
    if fp8_dtype is None:
        fp8_dtype = infer_dtype(a_fp8, None)
    if out_dtype is None:
        if not isinstance(out, torch.Tensor):
            raise ValueError("out_dtype is required for raw-pointer outputs")
        out_dtype = dtype_to_ks(out.dtype)
    if b_layout not in ("kn", "nk"):
        raise ValueError("b_layout must be 'kn' or 'nk'")
    check(lib.ks_moe_grouped_gemm_fp8_blockwise(
        ptr(out, name="out"), ptr(a_fp8, name="a_fp8"), ptr(b_fp8, name="b_fp8"),
        f32_ptr(a_scale, name="a_scale"), f32_ptr(b_scale, name="b_scale"),
        i32_ptr(expert_offsets, name="expert_offsets"), int(num_experts), int(total_rows), int(n), int(k),
        int(block_n), int(block_k), 1 if b_layout == "nk" else 0, int(fp8_dtype), int(out_dtype),
        default_stream(stream, a_fp8)), "ks_moe_grouped_gemm_fp8_blockwise")
    return out
