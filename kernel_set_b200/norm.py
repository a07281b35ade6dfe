"""Out-parameter wrappers of the RMSNorm entry points; ``rms_norm`` has the
signature of ``bindings/python/kernel_set/norm.py:48-77`` of the reference
project, ``rms_norm_quant_fp8`` wraps the added symbol that fuses the 1 x 128
FP8 quantizer."""
from __future__ import annotations

from typing import Optional

import torch

from ._lib import check, lib
from ._tensor import TensorLike, default_stream, f32_ptr, infer_dtype, ptr


def _rows_cols(t: TensorLike, rows: Optional[int], cols: Optional[int]):
    if rows is not None and cols is not None:
        return int(rows), int(cols)
    if not isinstance(t, torch.Tensor) or t.dim() < 1:
        raise ValueError("rows and cols are required for raw-pointer arguments")
    last = t.shape[-1]
    lead = t.numel() // last if last else 0
    return (lead if rows is None else int(rows)), (last if cols is None else int(cols))


def rms_norm(out: TensorLike, input: TensorLike, weight: TensorLike, rows: Optional[int] = None,
             cols: Optional[int] = None, eps: float = 1e-6, dtype: Optional[int] = None,
             stream: TensorLike = None) -> TensorLike:
    """``out = (x / rms(x)) * weight``, ``rms(x) = sqrt(mean(x^2) + eps)``."""
    rows, cols = _rows_cols(input, rows, cols)
    dt = infer_dtype(input, dtype)
    check(lib.ks_rms_norm(ptr(out, name="out"), ptr(input, name="input"), ptr(weight, name="weight"), rows, cols,
                          float(eps), dt, default_stream(stream, input)), "ks_rms_norm")
    return out


def rms_norm_quant_fp8(out_fp8: TensorLike, out_scale: TensorLike, input: TensorLike, weight: TensorLike,
                       rows: Optional[int] = None, cols: Optional[int] = None, eps: float = 1e-6,
                       in_dtype: Optional[int] = None, fp8_dtype: Optional[int] = None, stream: TensorLike = None):
    """RMSNorm fused with the 1 x 128 FP8 quantizer: ``out_fp8 [rows, cols]``,
    ``out_scale [rows, cols/128]``. Returns ``(out_fp8, out_scale)``."""
    rows, cols = _rows_cols(input, rows, cols)
    dt = infer_dtype(input, in_dtype)
    if fp8_dtype is None:
        fp8_dtype = infer_dtype(out_fp8, None)
    check(lib.ks_rms_norm_quant_fp8(ptr(out_fp8, name="out_fp8"), f32_ptr(out_scale, name="out_scale"),
                                    ptr(input, name="input"), ptr(weight, name="weight"), rows, cols, float(eps), dt,
                                    int(fp8_dtype), default_stream(stream, input)), "ks_rms_norm_quant_fp8")
    return out_fp8, out_scale
