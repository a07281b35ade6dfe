"""Operator layer: the ``ks.dispatch.*`` signatures of the reference project
for the quantized-GEMM path, returning freshly allocated tensors.

The reference routes each op through a ranked chain of external providers and
falls back to its own library (``bindings/python/kernel_set/dispatch.py:215-232``,
adapters in ``backends/_registry.py:464-492, 723-731, 1040-1046``). Here the
chain has exactly one entry, this library; the introspection helpers keep
their names and report it. ``_gpu`` / ``_dtype`` keyword arguments, which the
reference router consumes for provider selection (``dispatch.py:218-219``),
are accepted and ignored.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, List, Optional

import torch

from . import gemm as _gemm
from . import moe as _moe
from . import quant as _quant
from .enums import DType

KERNEL_SET = "kernel-set"

__all__ = [
    "fp8_gemm_blockwise", "per_token_group_quant", "per_token_group_quant_fp8", "w4a16", "moe",
    "which", "which_provider", "available", "providers", "ops", "chain", "Backend", "select",
    "resolve_sm", "reset_cache", "KERNEL_SET",
]


def _strip_router_kwargs(kw: dict) -> dict:
    kw.pop("_gpu", None)
    kw.pop("_dtype", None)
    return kw


# --------------------------------------------------------------------------- #
# ops
# --------------------------------------------------------------------------- #
def fp8_gemm_blockwise(a8, b8, a_scale, b_scale, *, block_n=128, block_k=128, out_dtype=None,
                       b_layout="kn", **kw):
    """FP8 block-scaled GEMM (1 x 128 activation scales, 128 x 128 weight-block
    scales, two-level fp32 accumulation). ``a8 [M,K]``; ``b_layout="kn"`` (the
    reference's own adapter, ``_registry.py:464-476``): ``b8 [K,N]``, ``b_scale
    [K/bk, N/bn]``; ``b_layout="nk"`` (what the reference's DeepGEMM adapter
    takes, ``_registry.py:416-424``): ``b8 [N,K]``, ``b_scale [N/bn, K/bk]``.
    The layout is never guessed from shapes. Returns ``[M,N]``, bf16 by default."""
    _strip_router_kwargs(kw)
    m, k = a8.shape
    n = b8.shape[1] if b_layout == "kn" else b8.shape[0]
    out = torch.empty(m, n, device=a8.device, dtype=out_dtype or torch.bfloat16)
    _gemm.gemm_fp8_blockwise(out, a8, b8, a_scale, b_scale, m=m, n=n, k=k, block_n=block_n, block_k=block_k,
                             b_layout=b_layout)
    return out


def per_token_group_quant(x, *, group_size=128, fp8_dtype=None, **kw):
    """1 x ``group_size`` dynamic FP8 activation quantization; returns
    ``(fp8_out [rows, cols], fp32_scale [rows, ceil(cols/group_size)])``
    (reference adapter ``_registry.py:479-492``)."""
    _strip_router_kwargs(kw)
    rows, cols = x.shape
    ngroups = (cols + group_size - 1) // group_size
    fp8 = DType(fp8_dtype) if fp8_dtype is not None else DType.F8E4M3
    tdt = torch.float8_e5m2 if fp8 == DType.F8E5M2 else torch.float8_e4m3fn
    out = torch.empty(rows, cols, device=x.device, dtype=tdt)
    scale = torch.empty(rows, ngroups, device=x.device, dtype=torch.float32)
    _quant.quantize_fp8_group(out, scale, x, rows=rows, cols=cols, group_size=group_size, fp8_dtype=fp8)
    return out, scale


# Name used by the reference's provider adapters for the same op
# (backends/_quant_ext.py:271-322).
per_token_group_quant_fp8 = per_token_group_quant


def w4a16(a, b_packed, scales, zeros, *, group_size=128, bias=None, **kw):
    """int4 weight-only GEMM: ``a [M,K]`` f16/bf16, ``b_packed`` uint8
    ``[K/2,N]``, ``scales``/``zeros`` ``[K/group_size,N]`` (``zeros`` may be
    ``None``). Returns ``[M,N]`` in ``a.dtype`` (reference adapter
    ``_registry.py:723-731``)."""
    _strip_router_kwargs(kw)
    m, k = a.shape
    n = scales.shape[1]
    c = torch.empty(m, n, device=a.device, dtype=a.dtype)
    _gemm.gemm_w4a16(c, a, b_packed, scales, zeros, m=m, n=n, k=k, group_size=group_size, bias=bias)
    return c


def moe(a, b, expert_offsets=None, *, num_experts=None, n, k, a_scale=None, b_scale=None, b_layout="nk",
        block_n=128, block_k=128, out_dtype=None, masked_m=None, expected_m=None, **kw):
    """Grouped expert GEMM over rows sorted by expert.

    Without scales this is the reference's own form (``_registry.py:1040-1046``):
    ``b [E,K,N]``, output in ``a.dtype``. With ``a_scale`` and ``b_scale`` it is
    the block-scaled FP8 form the reference hands to external providers
    (``_registry.py:1677-1700``): ``b [E,N,K]`` by default, bf16 output."""
    _strip_router_kwargs(kw)
    if masked_m is not None:
        # masked layout (``_registry.py:1686-1689``): a [E, max_m, K], out [E, max_m, N];
        # ``expected_m`` is a tuning hint of the external provider and is not needed here
        if a_scale is None or b_scale is None:
            raise ValueError("the masked layout needs a_scale and b_scale")
        e, max_m = a.shape[0], a.shape[1]
        out = torch.empty(e, max_m, n, device=a.device, dtype=out_dtype or torch.bfloat16)
        _moe.grouped_gemm_fp8_blockwise_masked(out, a, b, a_scale, b_scale, masked_m, e, max_m, n, k,
                                               block_n=block_n, block_k=block_k, b_layout=b_layout)
        return out
    if num_experts is None:
        num_experts = expert_offsets.shape[0] - 1
    total_rows = a.shape[0]
    if (a_scale is None) != (b_scale is None):
        raise ValueError("a_scale and b_scale must be given together")
    if a_scale is None:
        c = torch.empty(total_rows, n, device=a.device, dtype=a.dtype)
        _moe.grouped_gemm(c, a, b, expert_offsets, num_experts, total_rows, n, k)
        return c
    out = torch.empty(total_rows, n, device=a.device, dtype=out_dtype or torch.bfloat16)
    _moe.grouped_gemm_fp8_blockwise(out, a, b, a_scale, b_scale, expert_offsets, num_experts, total_rows, n, k,
                                    block_n=block_n, block_k=block_k, b_layout=b_layout)
    return out


# --------------------------------------------------------------------------- #
# introspection: one provider per op
# --------------------------------------------------------------------------- #
@dataclass(frozen=True)
class Provider:
    name: str
    rank: int
    min_sm: int
    dtypes: str
    note: str
    call: Callable


OPS: Dict[str, Provider] = {
    "fp8_gemm_blockwise": Provider(KERNEL_SET, 1, 100, "fp8", "tcgen05 kind::f8f6f4, TMEM partials, fp32 promotion",
                                   fp8_gemm_blockwise),
    "per_token_group_quant": Provider(KERNEL_SET, 1, 100, "fp32,fp16,bf16->fp8", "IEEE-division group quantizer",
                                      per_token_group_quant),
    "w4a16": Provider(KERNEL_SET, 1, 100, "fp16,bf16", "int4 group-wise weight-only GEMM", w4a16),
    "moe": Provider(KERNEL_SET, 1, 100, "fp32,fp16,bf16,fp8", "grouped GEMM, optional fp8 block scales", moe),
}
OP_ORDER: List[str] = list(OPS)


def reset_cache() -> None:
    """Kept for source compatibility; there is no selection cache to drop."""


def resolve_sm(gpu=None) -> Optional[int]:
    """SM version of ``gpu`` (an int like 100, a name containing "b200"), or of
    the current CUDA device; ``None`` when neither is available."""
    if isinstance(gpu, int):
        return gpu
    if isinstance(gpu, str):
        return 100 if "b200" in gpu.lower() or "sm100" in gpu.lower().replace("_", "") else None
    if torch.cuda.is_available():
        major, minor = torch.cuda.get_device_capability()
        return major * 10 + minor
    return None


def _known(op: str) -> Provider:
    try:
        return OPS[op]
    except KeyError:
        raise KeyError(f"unknown dispatch op {op!r}; known: {', '.join(OP_ORDER)}") from None


def select(op: str, gpu=None, dtype=None) -> Provider:
    return _known(op)


class Backend:
    """A bound op: ``Backend("w4a16")(a, b, s, z)``; ``.name`` is the provider."""

    __slots__ = ("op", "gpu", "dtype", "_provider")

    def __init__(self, op: str, gpu=None, dtype=None):
        self.op, self.gpu, self.dtype = op, gpu, dtype
        self._provider = select(op, gpu, dtype)

    @property
    def name(self) -> str:
        return self._provider.name

    @property
    def provider(self) -> Provider:
        return self._provider

    def __call__(self, *args, **kwargs):
        return self._provider.call(*args, **kwargs)

    def __repr__(self) -> str:
        return f"<Backend op={self.op!r} -> {self.name!r}>"


def which(op: str, gpu=None, dtype=None) -> str:
    return select(op, gpu, dtype).name


which_provider = which


def available(gpu=None, dtype=None) -> Dict[str, List[str]]:
    return {op: [OPS[op].name] for op in OP_ORDER}


def providers(op: str) -> List[str]:
    return [_known(op).name]


def ops() -> List[str]:
    return list(OP_ORDER)


def chain(op: str, gpu=None, dtype=None) -> List[dict]:
    p = _known(op)
    sm = resolve_sm(gpu)
    return [{"name": p.name, "rank": p.rank, "min_sm": p.min_sm, "dtypes": p.dtypes, "note": p.note,
             "selectable": sm is None or sm // 10 == 10, "is_kernel_set": True}]
