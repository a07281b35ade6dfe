"""Out-parameter wrappers of the quantized GEMM entry points; signatures of
``bindings/python/kernel_set/gemm.py`` of the reference project
(``gemm_w8a8`` ``:151-193``, ``gemm_w4a16`` ``:196-225``, ``gemm_fp8`` ``:228-280``,
``gemm_fp8_blockwise`` ``:313-362``)."""
from __future__ import annotations

from typing import Optional

import torch

from ._lib import check, lib
from ._tensor import TensorLike, default_stream, dtype_to_ks, f32_ptr, infer_dtype, ptr
from .enums import QuantMode


def _out_dtype(out, out_dtype, name):
    if out_dtype is not None:
        return int(out_dtype)
    if isinstance(out, torch.Tensor):
        return int(dtype_to_ks(out.dtype))
    raise ValueError(f"out_dtype is required for {name}")


def gemm_w8a8(c: TensorLike, a_i8: TensorLike, b_i8: TensorLike, a_scale: TensorLike, b_scale: TensorLike,
              m: int, n: int, k: int, bias: TensorLike = None, a_mode: int = QuantMode.PER_TOKEN,
              b_mode: int = QuantMode.PER_CHANNEL, out_dtype: int = None, stream: TensorLike = None) -> TensorLike:
    """W8A8 GEMM: int8 ``A [M,K]`` x int8 ``B [K,N]`` -> ``C [M,N]``;
    ``a_scale`` / ``b_scale`` fp32 ``[M]`` / ``[N]`` (or ``[1]``); ``bias [N]`` in
    the output dtype or ``None``."""
    odt = _out_dtype(c, out_dtype, "ks_gemm_w8a8")
    check(lib.ks_gemm_w8a8(ptr(c, name="c"), ptr(a_i8, name="a_i8"),
                           ptr(b_i8, name="b_i8"), f32_ptr(a_scale, name="a_scale"),
                           f32_ptr(b_scale, name="b_scale"), ptr(bias, name="bias"), int(m), int(n), int(k),
                           int(a_mode), int(b_mode), odt, default_stream(stream, a_i8)), "ks_gemm_w8a8")
    return c


def gemm_fp8(out: TensorLike, a_fp8: TensorLike, b_fp8: TensorLike, a_scale: TensorLike, b_scale: TensorLike,
             m: int, n: int, k: int, a_mode: int = QuantMode.PER_TOKEN, b_mode: int = QuantMode.PER_CHANNEL,
             fp8_dtype: int = None, out_dtype: int = None, stream: TensorLike = None) -> TensorLike:
    """FP8 GEMM ``C = (a_scale (x) b_scale) * (A_fp8 @ B_fp8)``: ``A [M,K]``,
    ``B [K,N]`` row-major, scales fp32 ``[M]`` / ``[N]`` (or ``[1]``)."""
    if fp8_dtype is None:
        fp8_dtype = infer_dtype(a_fp8, None)
    odt = _out_dtype(out, out_dtype, "ks_gemm_fp8")
    check(lib.ks_gemm_fp8(ptr(out, name="out"), ptr(a_fp8, name="a_fp8"), ptr(b_fp8, name="b_fp8"),
                          f32_ptr(a_scale, name="a_scale"), f32_ptr(b_scale, name="b_scale"), int(m), int(n), int(k),
                          int(a_mode), int(b_mode), int(fp8_dtype), odt, default_stream(stream, a_fp8)),
          "ks_gemm_fp8")
    return out


def gemm_w4a16(c: TensorLike, a: TensorLike, b_packed: TensorLike, scales: TensorLike, zeros: TensorLike,
               m: int, n: int, k: int, group_size: int, bias: TensorLike = None,
               dtype: Optional[int] = None, stream: TensorLike = None) -> TensorLike:
    """``C[M,N] = A[M,K] @ dequant(b_packed)`` (+ ``bias``): ``b_packed`` uint8
    ``[K/2,N]`` (even k in the low nibble), ``scales``/``zeros``
    ``[K/group_size,N]`` in the activation dtype, ``zeros`` may be ``None``."""
    dt = infer_dtype(a, dtype)
    check(lib.ks_gemm_w4a16(ptr(c, name="c"), ptr(a, name="a"), ptr(b_packed, name="b_packed"),
                            ptr(scales, name="scales"), ptr(zeros, name="zeros"), ptr(bias, name="bias"),
                            int(m), int(n), int(k), int(group_size), dt, default_stream(stream, a)),
          "ks_gemm_w4a16")
    return c


def gemm_w4a16_static_scratch(c: TensorLike, a: TensorLike, b_packed: TensorLike, scales: TensorLike,
                              zeros: TensorLike, m: int, n: int, k: int, group_size: int, bias: TensorLike = None,
                              dtype: Optional[int] = None, stream: TensorLike = None) -> TensorLike:
    """:func:`gemm_w4a16` through the entry point that never allocates: the
    kernel's split-K scratch is a fixed 16 MiB array inside the library. For
    hosts that forbid allocator calls at run time; shapes needing more scratch
    raise ``KernelSetError`` (UNSUPPORTED_SHAPE). All calls on a device share
    the array: do not let two of them overlap on the GPU."""
    dt = infer_dtype(a, dtype)
    check(lib.ks_gemm_w4a16_static_scratch(ptr(c, name="c"), ptr(a, name="a"), ptr(b_packed, name="b_packed"),
                                           ptr(scales, name="scales"), ptr(zeros, name="zeros"),
                                           ptr(bias, name="bias"), int(m), int(n), int(k), int(group_size), dt,
                                           default_stream(stream, a)), "ks_gemm_w4a16_static_scratch")
    return c


def gemm_fp8_blockwise(out: TensorLike, a_fp8: TensorLike, b_fp8: TensorLike, a_scale: TensorLike,
                       b_scale: TensorLike, m: int, n: int, k: int, block_n: int = 128, block_k: int = 128,
                       fp8_dtype: int = None, out_dtype: int = None, stream: TensorLike = None,
                       b_layout: str = "kn") -> TensorLike:
    """FP8 block-scaled GEMM. ``b_layout="kn"``: ``b_fp8 [K,N]``, ``b_scale
    [ceil(K/bk), ceil(N/bn)]`` (the reference ABI); ``b_layout="nk"``: ``b_fp8
    [N,K]``, ``b_scale [ceil(N/bn), ceil(K/bk)]`` (checkpoint layout)."""
    if fp8_dtype is None:
        fp8_dtype = infer_dtype(a_fp8, None)
    if out_dtype is None:
        if isinstance(out, torch.Tensor):
            out_dtype = dtype_to_ks(out.dtype)
        else:
            raise ValueError("out_dtype is required for ks_gemm_fp8_blockwise")
    if b_layout not in ("kn", "nk"):
        raise ValueError("b_layout must be 'kn' or 'nk'")
    fn, name = ((lib.ks_gemm_fp8_blockwise, "ks_gemm_fp8_blockwise") if b_layout == "kn"
                else (lib.ks_gemm_fp8_blockwise_nt, "ks_gemm_fp8_blockwise_nt"))
    check(fn(ptr(out, name="out"), ptr(a_fp8, name="a_fp8"), ptr(b_fp8, name="b_fp8"),
             f32_ptr(a_scale, name="a_scale"), f32_ptr(b_scale, name="b_scale"),
             int(m), int(n), int(k), int(block_n), int(block_k), int(fp8_dtype), int(out_dtype),
             default_stream(stream, out if not isinstance(out, int) else a_fp8)), name)
    return out


def gemm_fp8_blockwise_colscale(out: TensorLike, a_fp8: TensorLike, b_fp8: TensorLike, a_scale_t: TensorLike,
                                b_scale: TensorLike, m: int, n: int, k: int, a_scale_ld: Optional[int] = None,
                                fp8_dtype: int = None, out_dtype: int = None, stream: TensorLike = None,
                                b_layout: str = "kn") -> TensorLike:
    """The block-scaled GEMM with column-major activation scales ``a_scale_t
    [ceil(K/128), a_scale_ld]`` as ``quant.quantize_fp8_group_colscale`` writes
    them; everything else as :func:`gemm_fp8_blockwise`."""
    if fp8_dtype is None:
        fp8_dtype = infer_dtype(a_fp8, None)
    odt = _out_dtype(out, out_dtype, "ks_gemm_fp8_blockwise_colscale")
    if b_layout not in ("kn", "nk"):
        raise ValueError("b_layout must be 'kn' or 'nk'")
    if a_scale_ld is None:
        a_scale_ld = a_scale_t.shape[-1]
    check(lib.ks_gemm_fp8_blockwise_colscale(ptr(out, name="out"), ptr(a_fp8, name="a_fp8"), ptr(b_fp8, name="b_fp8"),
                                             f32_ptr(a_scale_t, name="a_scale_t"), int(a_scale_ld),
                                             f32_ptr(b_scale, name="b_scale"), int(m), int(n), int(k),
                                             1 if b_layout == "nk" else 0, int(fp8_dtype), odt,
                                             default_stream(stream, a_fp8)), "ks_gemm_fp8_blockwise_colscale")
    return out


def _ptr_array(items, name):
    import ctypes
    arr = (ctypes.c_void_p * len(items))()
    for i, t in enumerate(items):
        arr[i] = ptr(t, name=f"{name}[{i}]", allow_none=False)
    return arr


def gemm_fp8_blockwise_scatter(out_parts, a_fp8: TensorLike, b_fp8: TensorLike, a_scale: TensorLike,
                               b_scale: TensorLike, m: int, n: int, k: int, rows_per_part: int,
                               fp8_dtype: int = None, out_dtype: int = None, stream: TensorLike = None,
                               b_layout: str = "kn"):
    """The block-scaled GEMM whose row block ``b`` (``rows_per_part`` rows) is written to
    ``out_parts[b]``, a ``[rows_per_part, n]`` tensor (or raw address) that may live in
    another GPU's memory; see :func:`kernel_set_b200.parallel.FusedRowParallel`."""
    if fp8_dtype is None:
        fp8_dtype = infer_dtype(a_fp8, None)
    odt = _out_dtype(out_parts[0], out_dtype, "ks_gemm_fp8_blockwise_scatter")
    if b_layout not in ("kn", "nk"):
        raise ValueError("b_layout must be 'kn' or 'nk'")
    arr = _ptr_array(out_parts, "out_parts")
    check(lib.ks_gemm_fp8_blockwise_scatter(arr, len(out_parts), int(rows_per_part), ptr(a_fp8, name="a_fp8"),
                                            ptr(b_fp8, name="b_fp8"), f32_ptr(a_scale, name="a_scale"),
                                            f32_ptr(b_scale, name="b_scale"), int(m), int(n), int(k),
                                            1 if b_layout == "nk" else 0, int(fp8_dtype), odt,
                                            default_stream(stream, a_fp8)), "ks_gemm_fp8_blockwise_scatter")
    return out_parts


def sum_parts(dsts, parts: TensorLike, num_parts: int, rows: int, n: int, part_dtype: int = None,
              out_dtype: int = None, stream: TensorLike = None):
    """``sum(parts[q] for q)`` in fp32, rounded once, written to every tensor (or raw
    address) of ``dsts``; ``parts`` is ``[num_parts, rows, n]``."""
    pdt = infer_dtype(parts, part_dtype)
    odt = _out_dtype(dsts[0], out_dtype, "ks_sum_parts")
    arr = _ptr_array(dsts, "dsts")
    check(lib.ks_sum_parts(arr, len(dsts), ptr(parts, name="parts"), int(num_parts), int(rows), int(n), pdt, odt,
                           default_stream(stream, parts)), "ks_sum_parts")
    return dsts
