"""torch tensor -> (device pointer, dtype id, stream) marshalling.

Same rules as ``bindings/python/kernel_set/_tensor.py`` of the reference
project: tensors must be CUDA and contiguous (``ValueError`` otherwise,
``_tensor.py:155-165``); raw ``int`` addresses are accepted when the dtype is
given explicitly; the stream defaults to torch's current stream of the
reference tensor's device (``:205-219``); dtype map ``:81-93``.
"""
from __future__ import annotations

import ctypes
from typing import Any, Optional

import torch

from . import _lib

TensorLike = Any

TORCH_TO_KS = {
    torch.float32: _lib.KS_DTYPE_F32,
    torch.float16: _lib.KS_DTYPE_F16,
    torch.bfloat16: _lib.KS_DTYPE_BF16,
    torch.float64: _lib.KS_DTYPE_F64,
    torch.int64: _lib.KS_DTYPE_I64,
    torch.int32: _lib.KS_DTYPE_I32,
    torch.int8: _lib.KS_DTYPE_I8,
    torch.uint8: _lib.KS_DTYPE_U8,
    torch.float8_e4m3fn: _lib.KS_DTYPE_F8E4M3,
    torch.float8_e5m2: _lib.KS_DTYPE_F8E5M2,
}
KS_TO_TORCH = {v: k for k, v in TORCH_TO_KS.items()}


def dtype_to_ks(torch_dtype) -> int:
    try:
        return TORCH_TO_KS[torch_dtype]
    except KeyError:
        raise ValueError(f"torch dtype {torch_dtype!r} has no kernel_set equivalent") from None


def ks_to_torch_dtype(ks_dtype: int):
    try:
        return KS_TO_TORCH[int(ks_dtype)]
    except KeyError:
        raise ValueError(f"ks_dtype {ks_dtype} has no torch equivalent") from None


def ptr(obj: TensorLike, *, name: str = "tensor", allow_none: bool = True) -> int:
    """Raw device address of ``obj`` (tensor, int, or ``None`` -> 0)."""
    if obj is None:
        if allow_none:
            return 0
        raise ValueError(f"{name} must not be None")
    if isinstance(obj, int):
        return obj
    if isinstance(obj, torch.Tensor):
        if not obj.is_cuda:
            raise ValueError(f"{name} must be a CUDA tensor (got device {obj.device}); "
                             "kernel_set operates on device memory")
        if not obj.is_contiguous():
            raise ValueError(f"{name} must be contiguous; call .contiguous() first")
        return obj.data_ptr()
    dp = getattr(obj, "data_ptr", None)
    if callable(dp):
        return int(dp())
    raise TypeError(f"{name} must be a torch.Tensor, an int device pointer, or expose data_ptr(); "
                    f"got {type(obj).__name__}")


def f32_ptr(obj: TensorLike, *, name: str):
    return ctypes.cast(ptr(obj, name=name), ctypes.POINTER(ctypes.c_float))


def i32_ptr(obj: TensorLike, *, name: str):
    return ctypes.cast(ptr(obj, name=name), ctypes.POINTER(ctypes.c_int32))


def stream_ptr(stream: TensorLike) -> int:
    if stream is None:
        return 0
    if isinstance(stream, int):
        return stream
    if isinstance(stream, str) and stream == "current":
        return torch.cuda.current_stream().cuda_stream
    if isinstance(stream, torch.cuda.Stream):
        return stream.cuda_stream
    cs = getattr(stream, "cuda_stream", None)
    if cs is not None:
        return int(cs)
    raise TypeError(f"stream must be None, an int, 'current', or a torch.cuda.Stream; got {type(stream).__name__}")


def default_stream(stream: TensorLike, reference: TensorLike = None) -> int:
    if stream is not None:
        return stream_ptr(stream)
    if isinstance(reference, torch.Tensor) and reference.is_cuda:
        return torch.cuda.current_stream(reference.device).cuda_stream
    return 0


def infer_dtype(reference: TensorLike, dtype: Optional[int]) -> int:
    if dtype is not None:
        return int(dtype)
    if isinstance(reference, torch.Tensor):
        return dtype_to_ks(reference.dtype)
    raise ValueError("dtype must be given explicitly for raw-pointer arguments")
