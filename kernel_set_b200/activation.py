"""Out-parameter wrappers of the SwiGLU entry points with the signatures of
``bindings/python/kernel_set/activation.py`` of the reference project
(``swiglu``, ``swiglu_packed`` :121-143); ``swiglu_packed_quant_fp8`` wraps the
added symbol that fuses the 1 x 128 FP8 quantizer."""
from __future__ import annotations

from typing import Optional

import torch

from ._lib import check, lib
from ._tensor import TensorLike, default_stream, f32_ptr, infer_dtype, ptr


def _rows_inter(t: TensorLike, rows: Optional[int], inter: Optional[int]):
    if rows is not None and inter is not None:
        return int(rows), int(inter)
    if not isinstance(t, torch.Tensor) or t.dim() < 1:
        raise ValueError("rows and inter are required for raw-pointer arguments")
    last = t.shape[-1]
    lead = t.numel() // last if last else 0
    return (lead if rows is None else int(rows)), (last if inter is None else int(inter))


def swiglu(out: TensorLike, gate: TensorLike, up: TensorLike, rows: Optional[int] = None,
           inter: Optional[int] = None, dtype: Optional[int] = None, stream: TensorLike = None) -> TensorLike:
    """``out = silu(gate) * up``; all three ``[rows, inter]``."""
    rows, inter = _rows_inter(gate, rows, inter)
    dt = infer_dtype(gate, dtype)
    check(lib.ks_swiglu(ptr(out, name="out"), ptr(gate, name="gate"), ptr(up, name="up"), rows, inter, dt,
                        default_stream(stream, gate)), "ks_swiglu")
    return out


def swiglu_packed(out: TensorLike, input: TensorLike, rows: Optional[int] = None, inter: Optional[int] = None,
                  dtype: Optional[int] = None, stream: TensorLike = None) -> TensorLike:
    """Packed SwiGLU: ``input [rows, 2*inter]`` (gate = first half, up = second
    half); ``out [rows, inter]``."""
    if rows is None or inter is None:
        r, two_inter = _rows_inter(input, rows, None)
        rows = r if rows is None else int(rows)
        inter = two_inter // 2 if inter is None else int(inter)
    dt = infer_dtype(input, dtype)
    check(lib.ks_swiglu_packed(ptr(out, name="out"), ptr(input, name="input"), int(rows), int(inter), dt,
                               default_stream(stream, input)), "ks_swiglu_packed")
    return out


def swiglu_packed_quant_fp8(out_fp8: TensorLike, out_scale: TensorLike, input: TensorLike,
                            rows: Optional[int] = None, inter: Optional[int] = None, in_dtype: Optional[int] = None,
                            fp8_dtype: Optional[int] = None, stream: TensorLike = None):
    """Packed SwiGLU fused with the 1 x 128 FP8 quantizer: ``out_fp8 [rows,
    inter]``, ``out_scale [rows, inter/128]``. Returns ``(out_fp8, out_scale)``."""
    if rows is None or inter is None:
        r, two_inter = _rows_inter(input, rows, None)
        rows = r if rows is None else int(rows)
        inter = two_inter // 2 if inter is None else int(inter)
    dt = infer_dtype(input, in_dtype)
    if fp8_dtype is None:
        fp8_dtype = infer_dtype(out_fp8, None)
    check(lib.ks_swiglu_packed_quant_fp8(ptr(out_fp8, name="out_fp8"), f32_ptr(out_scale, name="out_scale"),
                                         ptr(input, name="input"), int(rows), int(inter), dt, int(fp8_dtype),
                                         default_stream(stream, input)), "ks_swiglu_packed_quant_fp8")
    return out_fp8, out_scale
