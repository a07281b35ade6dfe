"""CPU oracle of kernel-set's quantized-GEMM path. TEST INFRASTRUCTURE ONLY.

This module restates, with torch on the CPU, the arithmetic the reference
project itself uses to judge these ops (its torch statements in
``benchmarks/bench.py``). It exists so that tests, the smoke check and the
CPU-baseline leg of the benchmark have something to compare the CUDA library
against. Nothing in the product path (``kernel_set_b200``) imports it.

Pinning: ``tests/golden/make_golden.py`` ran the reference's own functions in
the build container (``_make_fp8_blockwise_inputs`` directly; the w4a16, int4
dequant and grouped-GEMM checks of ``bench.py`` with this oracle standing in
for the library, each reporting a relative error of exactly 0) and froze the
resulting vectors under ``tests/golden``; ``tests/test_oracle_golden.py``
replays them. The reference ships no golden vectors of its own for this path.

Each function cites the reference lines it follows (paths relative to the
reference project's root).
"""
from __future__ import annotations

from typing import Optional, Sequence, Tuple

import torch

FP8_DTYPES = {"e4m3": torch.float8_e4m3fn, "e5m2": torch.float8_e5m2}
FP8_MAX = {"e4m3": 448.0, "e5m2": 57344.0}  # kernels/src/quant/quant_common.cuh:25-27
SCALE_FLOOR = 1e-12                          # kernels/src/quant/quant_common.cuh:33


# --------------------------------------------------------------------------- #
# quantizers
# --------------------------------------------------------------------------- #
def quantize_fp8_group(x: torch.Tensor, group_size: int = 128, fp8: str = "e4m3"
                       ) -> Tuple[torch.Tensor, torch.Tensor]:
    """1 x group_size dynamic FP8 quantization.

    scale: benchmarks/bench.py:2339-2344 (``amax / 448`` in fp32, floor 1e-12);
    codes: benchmarks/bench.py:1454-1457 (``(x / scale).to(fp8)``, a true
    division, RNE). The last group of a row may be short
    (kernels/src/quant/quant_fp8_group.cu:49-50).
    Returns (codes [rows, cols] fp8, scale [rows, ceil(cols/gs)] fp32)."""
    xf = x.float()
    rows, cols = xf.shape
    qmax = FP8_MAX[fp8]
    scales = []
    out = torch.empty(rows, cols, dtype=FP8_DTYPES[fp8])
    for start in range(0, cols, group_size):
        group = xf[:, start:start + group_size]
        sc = (group.abs().amax(dim=1) / qmax).clamp_min(SCALE_FLOOR)
        scales.append(sc)
        out[:, start:start + group_size] = (group / sc[:, None]).to(FP8_DTYPES[fp8])
    return out, torch.stack(scales, dim=1)


def quantize_weight_blocks(w_kn: torch.Tensor, block_n: int = 128, block_k: int = 128, fp8: str = "e4m3"
                           ) -> Tuple[torch.Tensor, torch.Tensor]:
    """block_k x block_n weight-block quantization of a [K, N] matrix, the input
    preparation of benchmarks/bench.py:1447-1461. Returns (b8 [K,N], b_scale
    [ceil(K/bk), ceil(N/bn)])."""
    k, n = w_kn.shape
    wf = w_kn.float()
    nkb, nnb = -(-k // block_k), -(-n // block_n)
    scale = torch.empty(nkb, nnb, dtype=torch.float32)
    b8 = torch.empty(k, n, dtype=FP8_DTYPES[fp8])
    for kb in range(nkb):
        for nb in range(nnb):
            blk = wf[kb * block_k:(kb + 1) * block_k, nb * block_n:(nb + 1) * block_n]
            s = (blk.abs().amax() / FP8_MAX[fp8]).clamp_min(SCALE_FLOOR)
            scale[kb, nb] = s
            b8[kb * block_k:(kb + 1) * block_k, nb * block_n:(nb + 1) * block_n] = (blk / s).to(FP8_DTYPES[fp8])
    return b8, scale


# --------------------------------------------------------------------------- #
# FP8 block-scaled GEMM
# --------------------------------------------------------------------------- #
def _expand(scale: torch.Tensor, block: int, size: int, dim: int) -> torch.Tensor:
    return scale.repeat_interleave(block, dim=dim).narrow(dim, 0, size)


def dequantize_a(a8: torch.Tensor, a_scale: torch.Tensor, block_k: int = 128, dtype=torch.float32) -> torch.Tensor:
    """a8 [M,K] * a_scale [M, K/bk] broadcast over each strip (bench.py:1462-1465)."""
    return a8.to(dtype) * _expand(a_scale.to(dtype), block_k, a8.shape[1], 1)


def dequantize_b(b8: torch.Tensor, b_scale: torch.Tensor, block_n: int = 128, block_k: int = 128,
                 layout: str = "kn", dtype=torch.float32) -> torch.Tensor:
    """Block-dequantized weight as [K, N] (bench.py:1466-1469). ``layout="nk"``
    takes b8 [N,K] with b_scale [N/bn, K/bk]."""
    if layout == "nk":
        b8, b_scale = b8.t(), b_scale.t()
    k, n = b8.shape
    s = _expand(_expand(b_scale.to(dtype), block_k, k, 0), block_n, n, 1)
    return b8.to(dtype) * s


def fp8_gemm_blockwise(a8, b8, a_scale, b_scale, block_n: int = 128, block_k: int = 128, layout: str = "kn",
                       out_dtype: Optional[torch.dtype] = torch.bfloat16, acc=torch.float32) -> torch.Tensor:
    """Dequantize both operands, then one full-precision matmul
    (bench.py:1462-1470 and :1502). ``out_dtype=None`` returns the un-rounded
    accumulator; ``acc=torch.float64`` bounds the oracle's own rounding."""
    ref = dequantize_a(a8, a_scale, block_k, acc) @ dequantize_b(b8, b_scale, block_n, block_k, layout, acc)
    return ref if out_dtype is None else ref.to(out_dtype)


def fp8_gemm_blockwise_two_level(a8, b8, a_scale, b_scale, block_n: int = 128, block_k: int = 128,
                                 layout: str = "kn") -> torch.Tensor:
    """The algebra of the reference kernel, kernels/src/gemm/gemm_fp8_blockwise.cu:107-150:
    an fp32 inner product per K-block, folded in with ``part * (as * bs)``.
    Returns fp32. Used to show that kernel algebra and torch statement agree
    to accumulation-order noise."""
    if layout == "nk":
        b8, b_scale = b8.t(), b_scale.t()
    m, k = a8.shape
    n = b8.shape[1]
    af, bf = a8.float(), b8.float()
    out = torch.zeros(m, n, dtype=torch.float32)
    for kb in range(-(-k // block_k)):
        sl = slice(kb * block_k, min((kb + 1) * block_k, k))
        part = af[:, sl] @ bf[sl, :]
        bs = _expand(b_scale[kb:kb + 1].float(), block_n, n, 1)
        out += part * (a_scale[:, kb:kb + 1].float() * bs)
    return out


# --------------------------------------------------------------------------- #
# int4 formats
# --------------------------------------------------------------------------- #
def unpack_int4_words(qweight: torch.Tensor) -> torch.Tensor:
    """int32 [K/8, N] -> codes int32 [K, N]; code of k = 8*row + j is bits
    4j..4j+3 (bench.py:2469-2472, kernels/src/quant/dequant_int4.cu:46-50)."""
    k = qweight.shape[0] * 8
    kk = torch.arange(k)
    word = qweight[kk >> 3]
    shift = ((kk & 7) * 4).view(k, 1)
    return (word >> shift) & 0xF


def pack_int4_words(codes: torch.Tensor) -> torch.Tensor:
    """Inverse of :func:`unpack_int4_words` (codes [K, N] in 0..15, K % 8 == 0)."""
    k, n = codes.shape
    c = codes.to(torch.int64).view(k // 8, 8, n)
    word = torch.zeros(k // 8, n, dtype=torch.int64)
    for j in range(8):
        word |= c[:, j, :] << (4 * j)
    word = torch.where(word >= 2 ** 31, word - 2 ** 32, word)
    return word.to(torch.int32)


def unpack_int4_bytes(b_packed: torch.Tensor) -> torch.Tensor:
    """uint8 [K/2, N] -> codes [K, N]; even k in the low nibble
    (bench.py:1275-1281, kernels/src/gemm/gemm_w4a16.cu:43-48)."""
    k = b_packed.shape[0] * 2
    kk = torch.arange(k)
    byte = b_packed[kk >> 1].to(torch.int32)
    return torch.where((kk & 1).view(k, 1).bool(), (byte >> 4) & 0xF, byte & 0xF)


def pack_int4_bytes(codes: torch.Tensor) -> torch.Tensor:
    """codes [K, N] -> uint8 [K/2, N] (kernels/src/quant/repack_int4.cu:16-32)."""
    c = codes.to(torch.int32)
    return (c[0::2] | (c[1::2] << 4)).to(torch.uint8)


def repack_int4(qweight: torch.Tensor, perm: Optional[torch.Tensor] = None) -> torch.Tensor:
    """int32 [K/8, N] -> uint8 [K/2, N] (kernels/src/quant/repack_int4.cu:10-34).
    ``perm``: row k' of the result is row perm[k'] of the source, the meaning the
    argument has in the provider the reference routes the op to
    (bindings/python/kernel_set/backends/_quant_ext.py:217-227); the reference's
    own kernel refuses it (repack_int4.cu:52-53)."""
    codes = unpack_int4_words(qweight)
    if perm is not None:
        codes = codes[perm.long()]
    return pack_int4_bytes(codes)


# Checkpoint formats. The reference holds no code for them (its documentation
# names the gap, docs/QUANT_OPERATORS.md:71-75, 165); these are the published
# layouts of the GPTQ and AWQ file formats, pinned in tests/golden against the
# packers of the provider the reference routes the op to.
AWQ_ORDER = (0, 2, 4, 6, 1, 3, 5, 7)     # nibble i of a word holds column 8c + AWQ_ORDER[i]


def _to_i32(word: torch.Tensor) -> torch.Tensor:
    return torch.where(word >= 2 ** 31, word - 2 ** 32, word).to(torch.int32)


def pack_cols(values: torch.Tensor, order: Sequence[int] = tuple(range(8))) -> torch.Tensor:
    """[R, N] codes -> int32 [R, N/8]; nibble i of word c holds column 8c + order[i]."""
    r, n = values.shape
    v = values.to(torch.int64).view(r, n // 8, 8)
    word = torch.zeros(r, n // 8, dtype=torch.int64)
    for i, col in enumerate(order):
        word |= (v[:, :, col] & 0xF) << (4 * i)
    return _to_i32(word)


def unpack_cols(words: torch.Tensor, order: Sequence[int] = tuple(range(8))) -> torch.Tensor:
    """Inverse of :func:`pack_cols`: int32 [R, N/8] -> codes int32 [R, N]."""
    r, nc = words.shape
    w = words.to(torch.int64) & 0xFFFFFFFF
    out = torch.zeros(r, nc, 8, dtype=torch.int32)
    for i, col in enumerate(order):
        out[:, :, col] = ((w >> (4 * i)) & 0xF).to(torch.int32)
    return out.view(r, nc * 8)


def gptq_checkpoint(codes: torch.Tensor, zeros: torch.Tensor, zero_offset: int = 1):
    """codes [K, N], zero-points [G, N] -> (qweight [K/8, N], qzeros [G, N/8]) as a GPTQ
    file holds them: codes packed along K, zero-points minus ``zero_offset`` along N."""
    return pack_int4_words(codes), pack_cols(zeros - zero_offset)


def awq_checkpoint(codes: torch.Tensor, zeros: torch.Tensor):
    """codes [K, N], zero-points [G, N] -> (qweight [K, N/8], qzeros [G, N/8]) as an AWQ
    (GEMM format) file holds them: both packed along N in the interleaved order."""
    return pack_cols(codes, AWQ_ORDER), pack_cols(zeros, AWQ_ORDER)


def import_int4_weight(qweight: torch.Tensor, source: str, packing: str = "bytes",
                       perm: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Checkpoint qweight -> uint8 [K/2, N] (``packing="bytes"``) or int32 [K/8, N]
    (``"words"``); ``perm`` as in :func:`repack_int4`."""
    codes = unpack_int4_words(qweight) if source == "gptq" else unpack_cols(qweight, AWQ_ORDER)
    if perm is not None:
        codes = codes[perm.long()]
    return pack_int4_bytes(codes) if packing == "bytes" else pack_int4_words(codes)


def import_int4_zeros(qzeros: torch.Tensor, source: str, zero_offset: int, dtype=torch.float32) -> torch.Tensor:
    """Packed zero-points [G, N/8] -> [G, N] = code + zero_offset in ``dtype``."""
    codes = unpack_cols(qzeros) if source == "gptq" else unpack_cols(qzeros, AWQ_ORDER)
    return (codes + zero_offset).to(dtype)


def act_order_perm(g_idx: torch.Tensor) -> torch.Tensor:
    """The row order that makes the groups of an activation-ordered GPTQ layer
    contiguous: a stable argsort of g_idx."""
    return torch.argsort(g_idx.long(), stable=True).to(torch.int32)


def dequantize_int4(qweight: torch.Tensor, scales: torch.Tensor, zeros: torch.Tensor, group_size: int,
                    dtype=None) -> torch.Tensor:
    """(q - zero) * scale in fp32, rounded once to ``dtype`` (bench.py:2469-2476)."""
    dtype = dtype or scales.dtype
    codes = unpack_int4_words(qweight).float()
    g = torch.arange(codes.shape[0]) // group_size
    return ((codes - zeros.float()[g]) * scales.float()[g]).to(dtype)


# --------------------------------------------------------------------------- #
# W4A16
# --------------------------------------------------------------------------- #
def w4a16_weight(b_packed, scales, zeros, group_size: int) -> torch.Tensor:
    """The dequantized weight rounded to the activation dtype (bench.py:1275-1283)."""
    codes = unpack_int4_bytes(b_packed).float()
    k = codes.shape[0]
    gs = group_size if group_size > 0 else k
    g = torch.arange(k) // gs
    z = zeros.float()[g] if zeros is not None else 0.0
    return ((codes - z) * scales.float()[g]).to(scales.dtype)


def w4a16(a, b_packed, scales, zeros, group_size: int = 128, bias=None, out_dtype="same") -> torch.Tensor:
    """``(a.float() @ weight.float())`` with the weight of :func:`w4a16_weight`
    (bench.py:1282-1284); bias added in fp32 before the single output rounding
    (kernels/src/gemm/gemm_w4a16.cu:124-126). ``out_dtype=None`` returns fp32."""
    acc = a.float() @ w4a16_weight(b_packed, scales, zeros, group_size).float()
    if bias is not None:
        acc = acc + bias.float()
    if out_dtype is None:
        return acc
    return acc.to(a.dtype if out_dtype == "same" else out_dtype)


# --------------------------------------------------------------------------- #
# grouped GEMM / MoE
# --------------------------------------------------------------------------- #
def grouped_gemm(a, b, expert_offsets: Sequence[int], out_dtype="same") -> torch.Tensor:
    """Per-expert ``a[lo:hi].float() @ b[e].float()`` (bench.py:1593-1598); b [E,K,N]."""
    off = [int(v) for v in expert_offsets]
    dt = a.dtype if out_dtype == "same" else out_dtype
    ref = torch.zeros(a.shape[0], b.shape[2], dtype=torch.float32 if dt is None else dt)
    for e in range(len(off) - 1):
        lo, hi = off[e], off[e + 1]
        if hi > lo:
            r = a[lo:hi].float() @ b[e].float()
            ref[lo:hi] = r if dt is None else r.to(dt)
    return ref


def grouped_gemm_fp8_blockwise(a8, b8, a_scale, b_scale, expert_offsets: Sequence[int], block_n: int = 128,
                               block_k: int = 128, layout: str = "nk", out_dtype=torch.bfloat16) -> torch.Tensor:
    """The block-scaled product of :func:`fp8_gemm_blockwise` per expert over the
    offsets of :func:`grouped_gemm`. b8 [E,N,K] ("nk") or [E,K,N] ("kn")."""
    off = [int(v) for v in expert_offsets]
    n = b8.shape[1] if layout == "nk" else b8.shape[2]
    ref = torch.zeros(a8.shape[0], n, dtype=torch.float32 if out_dtype is None else out_dtype)
    for e in range(len(off) - 1):
        lo, hi = off[e], off[e + 1]
        if hi > lo:
            ref[lo:hi] = fp8_gemm_blockwise(a8[lo:hi], b8[e], a_scale[lo:hi], b_scale[e], block_n, block_k,
                                            layout, out_dtype)
    return ref


def gemm_fp8_scaled(a8, b8_kn, a_scale, b_scale, out_dtype=torch.bfloat16) -> torch.Tensor:
    """``(acc * a_scale) * b_scale`` with ``acc = A8.float() @ B8.float()``; scales
    ``[M]`` / ``[N]`` or one element (include/kernel_set/gemm.h:60-77,
    kernels/src/gemm/gemm_fp8.cu:147-153). ``out_dtype=None`` returns fp32."""
    acc = a8.float() @ b8_kn.float()
    ref = (acc * a_scale.float().reshape(-1, 1)) * b_scale.float().reshape(1, -1)
    return ref if out_dtype is None else ref.to(out_dtype)


def gemm_w8a8(a_i8, b_i8, a_scale, b_scale, bias=None, out_dtype=torch.bfloat16) -> torch.Tensor:
    """Exact integer product (in float64, as bench.py:1228-1232 does), then
    ``acc * a_scale * b_scale`` (+ bias) in fp32 (kernels/src/gemm/gemm_w8a8.cu:134-141)."""
    acc = (a_i8.double() @ b_i8.double()).float()
    ref = acc * a_scale.float().reshape(-1, 1) * b_scale.float().reshape(1, -1)
    if bias is not None:
        ref = ref + bias.float()
    return ref if out_dtype is None else ref.to(out_dtype)


def moe_route(logits: torch.Tensor, top_k: int):
    """softmax -> top-k -> renormalise (bench.py:1555-1557). Returns (weights
    fp32 [T,k], expert ids int64 [T,k])."""
    probs = torch.softmax(logits.float(), dim=-1)
    w, i = torch.topk(probs, top_k, dim=-1)
    return w / w.sum(-1, keepdim=True), i


def sort_by_expert(expert_ids: torch.Tensor, num_experts: int):
    """Stable counting sort of the (token, slot) pairs by expert. Returns
    (order [T*k] indices into the flattened pairs, offsets int32 [E+1])."""
    flat = expert_ids.reshape(-1)
    order = torch.sort(flat, stable=True).indices
    counts = torch.bincount(flat, minlength=num_experts)
    offsets = torch.zeros(num_experts + 1, dtype=torch.int32)
    offsets[1:] = torch.cumsum(counts, 0).to(torch.int32)
    return order, offsets


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """``(x * rsqrt(mean(x^2) + eps)).to(dtype) * weight`` (bench.py:877-879)."""
    f = x.float()
    return (f * torch.rsqrt(f.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype) * weight


def moe_permute(x: torch.Tensor, sorted_token_ids: torch.Tensor, top_k: int) -> torch.Tensor:
    """Gather rows by the permutation: row r of the result is token
    ``sorted_token_ids[r] // top_k`` (bench.py:2546-2548)."""
    return x.index_select(0, sorted_token_ids.to(torch.int64) // top_k)


def moe_unpermute(permuted: torch.Tensor, sorted_token_ids: torch.Tensor, weights: torch.Tensor, num_tokens: int,
                  top_k: int, out_dtype="same") -> torch.Tensor:
    """``out[token] = sum_k weight[token,k] * permuted[pos(token,k)]`` as a weighted
    scatter-add in fp32 (bench.py:2570-2579). ``out_dtype=None`` returns fp32."""
    ids = sorted_token_ids.to(torch.int64)
    dst_tok, slot = ids // top_k, ids % top_k
    contrib = permuted.float() * weights[dst_tok, slot].unsqueeze(1).float()
    ref = torch.zeros(num_tokens, permuted.shape[1], dtype=torch.float32)
    ref.index_add_(0, dst_tok, contrib)
    if out_dtype is None:
        return ref
    return ref.to(permuted.dtype if out_dtype == "same" else out_dtype)


def swiglu(gate: torch.Tensor, up: torch.Tensor, out_dtype="same") -> torch.Tensor:
    """``silu(gate.float()) * up.float()`` rounded once (bench.py:957-958)."""
    ref = torch.nn.functional.silu(gate.float()) * up.float()
    if out_dtype is None:
        return ref
    return ref.to(gate.dtype if out_dtype == "same" else out_dtype)


def swiglu_packed(x: torch.Tensor, out_dtype="same") -> torch.Tensor:
    """Packed form: gate = x[:, :inter], up = x[:, inter:]
    (kernels/src/activation/gated_mlp.cu:91-117)."""
    inter = x.shape[1] // 2
    return swiglu(x[:, :inter], x[:, inter:], out_dtype)


# --------------------------------------------------------------------------- #
# error measures
# --------------------------------------------------------------------------- #
def rel_err_max(a: torch.Tensor, b: torch.Tensor) -> float:
    """max|a-b| / max|b| — the reference benchmark's gate (bench.py:847-852)."""
    a, b = a.detach().float(), b.detach().float()
    return (a - b).abs().max().item() / b.abs().max().clamp_min(1e-6).item()


def rel_frobenius(a: torch.Tensor, b: torch.Tensor) -> float:
    a, b = a.detach().double(), b.detach().double()
    return ((a - b).norm() / b.norm().clamp_min(1e-30)).item()


def bf16_ulp(x: torch.Tensor) -> torch.Tensor:
    """Spacing of bf16 at |x| (x is the un-rounded fp32 value): 2^(floor(log2|x|) - 7)."""
    ax = x.detach().abs().double().clamp_min(2.0 ** -126)
    return torch.pow(2.0, torch.floor(torch.log2(ax)) - 7)


def ulp_violations(out: torch.Tensor, ref32: torch.Tensor, ulps: float = 2.0, noise: Optional[torch.Tensor] = None
                   ) -> Tuple[int, int]:
    """Counts elements with |out - ref32| > ulps * ulp_bf16(ref32). Returns
    (violations, violations whose error is also above `noise`), where `noise`
    is an elementwise bound on accumulation-order noise; the second count
    ignores elements whose exact value is tiny next to the terms summed into it."""
    err = (out.detach().double() - ref32.detach().double()).abs()
    bad = err > ulps * bf16_ulp(ref32)
    n_bad = int(bad.sum())
    if noise is None:
        return n_bad, n_bad
    return n_bad, int((bad & (err > noise.double())).sum())
