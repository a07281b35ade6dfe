"""Out-parameter wrappers of the quantizer and int4 helpers; signatures of
``bindings/python/kernel_set/quant.py`` of the reference project
(``quantize_fp8_group`` ``:62-87``, ``dequantize_int4`` / ``repack_int4``
``:168-212``)."""
from __future__ import annotations

from typing import Optional

from ._lib import check, lib
from ._tensor import TensorLike, default_stream, f32_ptr, infer_dtype, ptr
from .enums import DType


def quantize_fp8_group(out: TensorLike, scale: TensorLike, input: TensorLike, rows: int, cols: int,
                       group_size: int = 128, in_dtype: Optional[int] = None,
                       fp8_dtype: int = DType.F8E4M3, stream: TensorLike = None):
    """1 x ``group_size`` dynamic FP8 quantization. ``out`` fp8 ``[rows, cols]``,
    ``scale`` fp32 ``[rows, ceil(cols/group_size)]``. Returns ``(out, scale)``."""
    dt = infer_dtype(input, in_dtype)
    check(lib.ks_quantize_fp8_group(ptr(out, name="out"), f32_ptr(scale, name="scale"), ptr(input, name="input"),
                                    int(rows), int(cols), int(group_size), dt, int(fp8_dtype),
                                    default_stream(stream, input)), "ks_quantize_fp8_group")
    return out, scale


def quantize_fp8_group_colscale(out: TensorLike, scale_t: TensorLike, input: TensorLike, rows: int, cols: int,
                                scale_ld: Optional[int] = None, in_dtype: Optional[int] = None,
                                fp8_dtype: int = DType.F8E4M3, stream: TensorLike = None):
    """1 x 128 FP8 quantization with the scales stored column-major:
    ``scale_t [cols/128, scale_ld]`` fp32, ``scale_t[g, r]`` = scale of row ``r``,
    group ``g`` (``scale_ld >= rows``; default: ``scale_t``'s row length).
    Returns ``(out, scale_t)``."""
    dt = infer_dtype(input, in_dtype)
    if scale_ld is None:
        scale_ld = scale_t.shape[-1]
    check(lib.ks_quantize_fp8_group_colscale(ptr(out, name="out"), f32_ptr(scale_t, name="scale_t"), int(scale_ld),
                                             ptr(input, name="input"), int(rows), int(cols), dt, int(fp8_dtype),
                                             default_stream(stream, input)), "ks_quantize_fp8_group_colscale")
    return out, scale_t


def dequantize_int4(out: TensorLike, qweight_packed: TensorLike, scales: TensorLike, zeros: TensorLike,
                    k: int, n: int, group_size: int, out_dtype: Optional[int] = None,
                    stream: TensorLike = None) -> TensorLike:
    """int32 ``[k/8, n]`` (nibble j of a word = code of k = 8*row + j) ->
    ``out [k, n]`` = ``(q - zeros) * scales``."""
    dt = infer_dtype(out, out_dtype)
    check(lib.ks_dequantize_int4(ptr(out, name="out"), ptr(qweight_packed, name="qweight_packed"),
                                 ptr(scales, name="scales"), ptr(zeros, name="zeros"),
                                 int(k), int(n), int(group_size), dt, default_stream(stream, out)),
          "ks_dequantize_int4")
    return out


def repack_int4(out_packed: TensorLike, qweight: TensorLike, perm: TensorLike, size_k: int, size_n: int,
                num_bits: int = 4, stream: TensorLike = None) -> TensorLike:
    """int32 ``[K/8, N]`` -> uint8 ``[K/2, N]`` (the layout ``gemm_w4a16`` reads)."""
    check(lib.ks_repack_int4(ptr(out_packed, name="out_packed"), ptr(qweight, name="qweight"),
                             ptr(perm, name="perm", allow_none=True), int(size_k), int(size_n), int(num_bits),
                             default_stream(stream, out_packed)), "ks_repack_int4")
    return out_packed
