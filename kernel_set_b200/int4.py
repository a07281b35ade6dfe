"""Import of GPTQ / AWQ int4 checkpoints into the layouts ``gemm.gemm_w4a16``
and ``quant.dequantize_int4`` read.

The reference project has no own kernel for this step: its documentation
names the re-layout as a gap (``docs/QUANT_OPERATORS.md:71-75, 165``), its
``ks_repack_int4`` refuses activation order (``kernels/src/quant/
repack_int4.cu:52-53``) and its dispatcher hands the op to external providers
(``bindings/python/kernel_set/backends/_quant_ext.py:217-241``). The formats:

  GPTQ  ``qweight [K/8, N]`` int32 (code of ``k = 8*row + j`` in bits
        ``4j..4j+3``), ``qzeros [G, N/8]`` int32 (column ``8c+j`` in bits
        ``4j..4j+3``; files of the first format version store ``zero - 1``),
        ``scales [G, N]``, ``g_idx [K]`` (group of each row; not ``k // gs``
        when the rows were quantised in activation order).
  AWQ   ``qweight [K, N/8]``, ``qzeros [G, N/8]`` int32 with column ``8c+j`` in
        nibble ``(0,4,1,5,2,6,3,7)[j]`` of word ``c``; ``scales [G, N]``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from . import gemm as _gemm
from ._lib import check, lib
from ._tensor import TensorLike, default_stream, dtype_to_ks, infer_dtype, ptr
from .enums import Int4Packing, Int4Source


def import_weight(out: TensorLike, qweight: TensorLike, size_k: int, size_n: int, source: int,
                  packing: int = Int4Packing.BYTES, perm: TensorLike = None, stream: TensorLike = None) -> TensorLike:
    """Codes of a checkpoint's ``qweight`` -> ``out`` in one of the library's two
    packings; ``perm`` (int32 ``[K]``): row ``k'`` of the result is row
    ``perm[k']`` of the source."""
    check(lib.ks_int4_import_weight(ptr(out, name="out"), ptr(qweight, name="qweight"), ptr(perm, name="perm"),
                                    int(size_k), int(size_n), int(source), int(packing),
                                    default_stream(stream, qweight)), "ks_int4_import_weight")
    return out


def import_zeros(zeros: TensorLike, qzeros: TensorLike, groups: int, size_n: int, source: int, zero_offset: int,
                 out_dtype: Optional[int] = None, stream: TensorLike = None) -> TensorLike:
    """Packed zero-points ``[G, N/8]`` -> ``zeros [G, N]`` = code + ``zero_offset``."""
    dt = infer_dtype(zeros, out_dtype)
    check(lib.ks_int4_import_zeros(ptr(zeros, name="zeros"), ptr(qzeros, name="qzeros"), int(groups), int(size_n),
                                   int(source), int(zero_offset), dt, default_stream(stream, qzeros)),
          "ks_int4_import_zeros")
    return zeros


def gather_columns(out: TensorLike, input: TensorLike, perm: TensorLike, rows: int, cols: int,
                   dtype: Optional[int] = None, stream: TensorLike = None) -> TensorLike:
    """``out[r, j] = input[r, perm[j]]``."""
    dt = infer_dtype(input, dtype)
    check(lib.ks_gather_columns(ptr(out, name="out"), ptr(input, name="input"), ptr(perm, name="perm"),
                                int(rows), int(cols), dt, default_stream(stream, input)), "ks_gather_columns")
    return out


@dataclass
class Int4Linear:
    """An imported layer: ``y = x[:, perm] @ dequant(b_packed)``."""
    b_packed: torch.Tensor            # uint8 [K/2, N]
    scales: torch.Tensor              # [G, N] in the activation dtype
    zeros: torch.Tensor               # [G, N] in the activation dtype
    perm: Optional[torch.Tensor]      # int32 [K] or None
    k: int
    n: int
    group_size: int

    def __call__(self, x: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
        m = x.shape[0]
        if self.perm is not None:
            x = gather_columns(torch.empty_like(x), x, self.perm, m, self.k)
        out = torch.empty(m, self.n, dtype=x.dtype, device=x.device)
        return _gemm.gemm_w4a16(out, x, self.b_packed, self.scales, self.zeros, m, self.n, self.k,
                                self.group_size, bias=bias)


def _finish(qweight, qzeros, scales, source, zero_offset, perm, dtype):
    k = qweight.shape[0] * (8 if source == Int4Source.GPTQ else 1)
    n = scales.shape[1]
    groups = scales.shape[0]
    if k % groups != 0:
        raise ValueError("K must be a multiple of the number of groups")
    dtype = dtype or scales.dtype
    b_packed = torch.empty(k // 2, n, dtype=torch.uint8, device=qweight.device)
    import_weight(b_packed, qweight.contiguous(), k, n, source, Int4Packing.BYTES, perm=perm)
    zeros = torch.empty(groups, n, dtype=dtype, device=qweight.device)
    import_zeros(zeros, qzeros.contiguous(), groups, n, source, zero_offset, out_dtype=dtype_to_ks(dtype))
    return Int4Linear(b_packed, scales.to(dtype).contiguous(), zeros, perm, k, n, k // groups)


def from_gptq(qweight: torch.Tensor, qzeros: torch.Tensor, scales: torch.Tensor,
              g_idx: Optional[torch.Tensor] = None, zero_offset: int = 1, dtype=None) -> Int4Linear:
    """A GPTQ layer. ``g_idx`` other than ``k // group_size`` (activation
    order) reorders the rows so that each group is contiguous; every group must
    then hold exactly ``group_size`` rows, which is how the format writes them."""
    perm = None
    if g_idx is not None:
        k = qweight.shape[0] * 8
        gs = k // scales.shape[0]
        trivial = torch.arange(k, device=g_idx.device, dtype=g_idx.dtype) // gs
        if not torch.equal(g_idx, trivial):
            if not torch.equal(torch.bincount(g_idx.long(), minlength=scales.shape[0]),
                               torch.full((scales.shape[0],), gs, device=g_idx.device)):
                raise ValueError("g_idx must name every group exactly group_size times")
            perm = torch.argsort(g_idx.long(), stable=True).to(torch.int32).contiguous()
    return _finish(qweight, qzeros, scales, Int4Source.GPTQ, zero_offset, perm, dtype)


def from_awq(qweight: torch.Tensor, qzeros: torch.Tensor, scales: torch.Tensor, dtype=None) -> Int4Linear:
    """An AWQ (GEMM format) layer."""
    return _finish(qweight, qzeros, scales, Int4Source.AWQ, 0, None, dtype)
