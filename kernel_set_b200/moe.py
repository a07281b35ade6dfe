"""Out-parameter wrappers of the mixture-of-experts entry points with the
signatures of ``bindings/python/kernel_set/moe.py`` of the reference project
(``gate_softmax_topk`` :42-71, ``compute_permutation`` :109-134, ``permute``
:137-159, ``unpermute`` :162-186, ``grouped_gemm`` :189-217);
``grouped_gemm_fp8_blockwise`` and ``permute_quant_fp8`` wrap added symbols."""
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


def gate_softmax_topk(out_weights: TensorLike, out_indices: TensorLike, logits: TensorLike, num_tokens: int,
                      num_experts: int, top_k: int, renormalize: bool = True, dtype: Optional[int] = None,
                      stream: TensorLike = None):
    """Softmax over experts then top-k. ``logits [num_tokens, num_experts]``;
    ``out_weights [num_tokens, top_k]`` fp32; ``out_indices [num_tokens, top_k]``
    int32. Returns ``(out_weights, out_indices)``."""
    dt = infer_dtype(logits, dtype)
    check(lib.ks_moe_gate_softmax_topk(f32_ptr(out_weights, name="out_weights"),
                                       i32_ptr(out_indices, name="out_indices"), ptr(logits, name="logits"),
                                       int(num_tokens), int(num_experts), int(top_k), 1 if renormalize else 0, dt,
                                       default_stream(stream, logits)), "ks_moe_gate_softmax_topk")
    return out_weights, out_indices


def compute_permutation(sorted_token_ids: TensorLike, expert_offsets: TensorLike, topk_indices: TensorLike,
                        num_tokens: int, num_experts: int, top_k: int, stream: TensorLike = None):
    """The permutation that groups (token, slot) pairs by expert.
    ``topk_indices [num_tokens, top_k]`` int32; ``sorted_token_ids
    [num_tokens*top_k]`` int32; ``expert_offsets [num_experts+1]`` int32.
    Returns ``(sorted_token_ids, expert_offsets)``."""
    check(lib.ks_moe_compute_permutation(i32_ptr(sorted_token_ids, name="sorted_token_ids"),
                                         i32_ptr(expert_offsets, name="expert_offsets"),
                                         i32_ptr(topk_indices, name="topk_indices"), int(num_tokens),
                                         int(num_experts), int(top_k), default_stream(stream, topk_indices)),
          "ks_moe_compute_permutation")
    return sorted_token_ids, expert_offsets


def permute(permuted: TensorLike, input: TensorLike, sorted_token_ids: TensorLike, num_tokens: int, top_k: int,
            hidden: int, dtype: Optional[int] = None, stream: TensorLike = None) -> TensorLike:
    """Gather rows of ``input [num_tokens, hidden]`` into ``permuted
    [num_tokens*top_k, hidden]`` following ``sorted_token_ids``."""
    dt = infer_dtype(input, dtype)
    check(lib.ks_moe_permute(ptr(permuted, name="permuted"), ptr(input, name="input"),
                             i32_ptr(sorted_token_ids, name="sorted_token_ids"), int(num_tokens), int(top_k),
                             int(hidden), dt, default_stream(stream, input)), "ks_moe_permute")
    return permuted


def permute_quant_fp8(out_fp8: TensorLike, out_scale: TensorLike, input: TensorLike, sorted_token_ids: TensorLike,
                      num_tokens: int, top_k: int, hidden: int, in_dtype: Optional[int] = None,
                      fp8_dtype: Optional[int] = None, stream: TensorLike = None):
    """``permute`` fused with the 1 x 128 FP8 quantizer. Returns ``(out_fp8, out_scale)``."""
    dt = infer_dtype(input, in_dtype)
    if fp8_dtype is None:
        fp8_dtype = infer_dtype(out_fp8, None)
    check(lib.ks_moe_permute_quant_fp8(ptr(out_fp8, name="out_fp8"), f32_ptr(out_scale, name="out_scale"),
                                       ptr(input, name="input"), i32_ptr(sorted_token_ids, name="sorted_token_ids"),
                                       int(num_tokens), int(top_k), int(hidden), dt, int(fp8_dtype),
                                       default_stream(stream, input)), "ks_moe_permute_quant_fp8")
    return out_fp8, out_scale


def unpermute(out: TensorLike, permuted: TensorLike, sorted_token_ids: TensorLike, routing_weights: TensorLike,
              num_tokens: int, top_k: int, hidden: int, dtype: Optional[int] = None,
              stream: TensorLike = None) -> TensorLike:
    """``out[token] = sum_k weight[token,k] * permuted[pos(token,k)]``."""
    dt = infer_dtype(permuted, dtype)
    check(lib.ks_moe_unpermute(ptr(out, name="out"), ptr(permuted, name="permuted"),
                               i32_ptr(sorted_token_ids, name="sorted_token_ids"),
                               f32_ptr(routing_weights, name="routing_weights"), int(num_tokens), int(top_k),
                               int(hidden), dt, default_stream(stream, permuted)), "ks_moe_unpermute")
    return out


def grouped_gemm_fp8_blockwise_masked(out: TensorLike, a_fp8: TensorLike, b_fp8: TensorLike, a_scale: TensorLike,
                                      b_scale: TensorLike, masked_m: TensorLike, num_experts: int, max_m: int,
                                      n: int, k: int, block_n: int = 128, block_k: int = 128, b_layout: str = "nk",
                                      fp8_dtype: Optional[int] = None, out_dtype: Optional[int] = None,
                                      stream: TensorLike = None) -> TensorLike:
    """The block-scaled grouped GEMM over the masked layout: ``a_fp8 [E, max_m,
    K]``, ``masked_m [E]`` int32 (device), ``out [E, max_m, N]``; expert ``e``
    computes its first ``masked_m[e]`` rows."""
    if fp8_dtype is None:
        fp8_dtype = infer_dtype(a_fp8, None)
    if out_dtype is None:
        if not isinstance(out, torch.Tensor):
            raise ValueError("out_dtype is required for raw-pointer outputs")
        out_dtype = dtype_to_ks(out.dtype)
    if b_layout not in ("kn", "nk"):
        raise ValueError("b_layout must be 'kn' or 'nk'")
    check(lib.ks_moe_grouped_gemm_fp8_blockwise_masked(
        ptr(out, name="out"), ptr(a_fp8, name="a_fp8"), ptr(b_fp8, name="b_fp8"),
        f32_ptr(a_scale, name="a_scale"), f32_ptr(b_scale, name="b_scale"), i32_ptr(masked_m, name="masked_m"),
        int(num_experts), int(max_m), int(n), int(k), int(block_n), int(block_k), 1 if b_layout == "nk" else 0,
        int(fp8_dtype), int(out_dtype), default_stream(stream, a_fp8)), "ks_moe_grouped_gemm_fp8_blockwise_masked")
    return out


def _ptr_array(items, name):
    import ctypes
    arr = (ctypes.c_void_p * len(items))()
    for i, t in enumerate(items):
        arr[i] = ptr(t, name=f"{name}[{i}]", allow_none=False)
    return arr


def dispatch_plan(dst_base: TensorLike, local_offsets: TensorLike, seg_start: TensorLike, ret_base: TensorLike,
                  counts: TensorLike, world: int, rank: int, experts_per_rank: int, stream: TensorLike = None):
    """From the all-gathered count matrix ``counts [world, world * experts_per_rank]`` int32:
    where this rank's rows land on their destination ranks (``dst_base``), the expert offsets
    of what it receives (``local_offsets``), and the (expert, source) segments with their way
    back (``seg_start``, ``ret_base``). All int32, on the device."""
    check(lib.ks_moe_dispatch_plan(i32_ptr(dst_base, name="dst_base"), i32_ptr(local_offsets, name="local_offsets"),
                                   i32_ptr(seg_start, name="seg_start"), i32_ptr(ret_base, name="ret_base"),
                                   i32_ptr(counts, name="counts"), int(world), int(rank), int(experts_per_rank),
                                   default_stream(stream, counts)), "ks_moe_dispatch_plan")
    return dst_base, local_offsets, seg_start, ret_base


def permute_quant_fp8_scatter(dst_fp8, dst_scale, capacity_rows: int, dst_base: TensorLike, expert_offsets: TensorLike,
                              num_experts: int, experts_per_rank: int, input: TensorLike,
                              sorted_token_ids: TensorLike, num_tokens: int, top_k: int, hidden: int,
                              in_dtype: Optional[int] = None, fp8_dtype: int = None, stream: TensorLike = None):
    """:func:`permute_quant_fp8` with every row written to its destination rank's buffer
    (``dst_fp8[d]`` / ``dst_scale[d]``: tensors or raw peer addresses) at its expert-major row."""
    from .enums import DType
    dt = infer_dtype(input, in_dtype)
    q = _ptr_array(dst_fp8, "dst_fp8")
    s = _ptr_array(dst_scale, "dst_scale")
    check(lib.ks_moe_permute_quant_fp8_scatter(q, s, len(dst_fp8), int(capacity_rows), i32_ptr(dst_base, name="dst_base"),
                                               i32_ptr(expert_offsets, name="expert_offsets"), int(num_experts),
                                               int(experts_per_rank), ptr(input, name="input"),
                                               i32_ptr(sorted_token_ids, name="sorted_token_ids"), int(num_tokens),
                                               int(top_k), int(hidden), dt,
                                               int(fp8_dtype if fp8_dtype is not None else DType.F8E4M3),
                                               default_stream(stream, input)), "ks_moe_permute_quant_fp8_scatter")


def scatter_rows(dst, dst_rows: int, src: TensorLike, capacity_rows: int, seg_start: TensorLike, ret_base: TensorLike,
                 segments: int, hidden: int, dtype: Optional[int] = None, stream: TensorLike = None):
    """Received row ``i`` of ``src`` goes back to row ``ret_base[j] + i - seg_start[j]`` of
    ``dst[j % world]`` (tensors or raw peer addresses), ``j`` the segment that holds ``i``."""
    dt = infer_dtype(src, dtype)
    arr = _ptr_array(dst, "dst")
    check(lib.ks_moe_scatter_rows(arr, len(dst), int(dst_rows), ptr(src, name="src"), int(capacity_rows),
                                  i32_ptr(seg_start, name="seg_start"), i32_ptr(ret_base, name="ret_base"),
                                  int(segments), int(hidden), dt, default_stream(stream, src)), "ks_moe_scatter_rows")
