"""Shared helpers of the test-suite: seeded inputs in the value distributions
of the benchmark configurations, generated on the CPU so that the oracle and
the CUDA library see identical bits, and the acceptance checks."""
from __future__ import annotations

import os

import numpy as np
import torch

import ks_oracle as orc

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def golden(name: str):
    return np.load(os.path.join(GOLDEN, name))


def from_bits16(arr, dtype):
    return torch.from_numpy(np.ascontiguousarray(arr)).view(dtype)


def from_u8(arr, dtype):
    return torch.from_numpy(np.ascontiguousarray(arr)).view(dtype)


def gen(seed: int) -> torch.Generator:
    g = torch.Generator()
    g.manual_seed(seed)
    return g


def w4a16_inputs(m, k, n, group_size=128, dtype=torch.bfloat16, seed=0, with_zeros=True):
    """Activations ~N(0,1); symmetric int4 in [-8,7] stored as code q+8 with
    zero-point 8.0; scales |N(0,0.02)|+1e-3 (the decode-sweep recipe)."""
    g = gen(seed)
    a = torch.randn(m, k, generator=g).to(dtype)
    q = torch.randint(-8, 8, (k, n), generator=g)
    codes = (q + 8).to(torch.int32)
    gs = group_size if group_size > 0 else k
    scales = (torch.randn(k // gs, n, generator=g).mul(0.02).abs() + 1e-3).to(dtype)
    zeros = torch.full((k // gs, n), 8.0).to(dtype) if with_zeros else None
    if not with_zeros:
        codes = torch.randint(0, 16, (k, n), generator=g).to(torch.int32)
    return a, codes, scales, zeros


def fp8_inputs(m, n, k, seed=0, block_n=128, block_k=128, fp8="e4m3", a_std=1.0, w_std=0.02):
    """A ~N(0,1) bf16 quantized in 1 x block_k groups; W ~N(0,0.02) quantized in
    block_k x block_n blocks (the DeepSeek-shape recipe). Returns CPU tensors:
    a8, a_scale, b8_kn [K,N], b_scale_kn [K/bk, N/bn]."""
    g = gen(seed)
    a = (torch.randn(m, k, generator=g) * a_std).to(torch.bfloat16)
    w_kn = torch.randn(k, n, generator=g) * w_std
    a8, a_s = orc.quantize_fp8_group(a, block_k, fp8)
    b8, b_s = orc.quantize_weight_blocks(w_kn, block_n, block_k, fp8)
    return a8, a_s, b8, b_s


def check_gemm(out: torch.Tensor, ref32: torch.Tensor, noise: torch.Tensor | None = None, what: str = "",
               frob_tol: float = 1e-3, ulps: float = 2.0):
    """Acceptance of a GEMM output against the oracle: relative Frobenius error
    <= 1e-3 against the oracle's output (its fp32 accumulator rounded once to
    the output type, as the reference's torch statement does; rounding alone
    puts any bf16 tensor ~1.5e-3 away from an fp32 one), and |err| <= 2 bf16
    ulp of the un-rounded fp32 oracle value for every element whose error is
    not explained by accumulation-order noise (`noise`, an elementwise bound;
    elements below it are counted and returned, never silently accepted)."""
    out_dtype = out.dtype
    out = out.detach().float().cpu()
    frob = orc.rel_frobenius(out, ref32.to(out_dtype).float())
    bad, bad_above_noise = orc.ulp_violations(out, ref32, ulps, noise)
    assert frob <= frob_tol, f"{what}: relative Frobenius error {frob:.3e} > {frob_tol}"
    assert bad_above_noise == 0, (f"{what}: {bad_above_noise} elements off by more than {ulps} bf16 ulp "
                                  f"(and above the accumulation noise floor); {bad} before the floor")
    return frob, bad


def accumulation_noise(a_abs: torch.Tensor, b_abs: torch.Tensor, k: int) -> torch.Tensor:
    """Elementwise bound on the difference between two fp32 summation orders of
    the same products: ~ sqrt(k) * eps32 * sum|a||b| (a loose statistical bound,
    4 standard deviations)."""
    eps = 2.0 ** -24
    return (a_abs.double() @ b_abs.double()).float() * (4.0 * eps * (k ** 0.5))


def block_quant_nk_device(w_nk: torch.Tensor):
    """128 x 128 block quantization of a [N,K] fp32 weight on its own device: the
    reference's input preparation (benchmarks/bench.py:1447-1461) written with
    tensor ops (the same arithmetic as orc.quantize_weight_blocks, which loops
    over blocks on the CPU). Returns (e4m3 [N,K], scales [N/128, K/128])."""
    n, k = w_nk.shape
    blocks = w_nk.view(n // 128, 128, k // 128, 128)
    scale = (blocks.abs().amax(dim=(1, 3)) / 448.0).clamp_min(1e-12)
    q = (blocks / scale[:, None, :, None]).to(torch.float8_e4m3fn).view(n, k)
    return q, scale.contiguous()


def quant_group_device(x: torch.Tensor, group: int = 128):
    """orc.quantize_fp8_group with tensor ops on the tensor's own device (cols % group == 0)."""
    rows, cols = x.shape
    xf = x.float().view(rows, cols // group, group)
    sc = (xf.abs().amax(dim=2) / 448.0).clamp_min(1e-12)
    return (xf / sc[:, :, None]).to(torch.float8_e4m3fn).view(rows, cols), sc.contiguous()


def fp8_window_reference(a8, a_s, b8_nk, b_s_nk, rows: slice, cols: slice):
    """Oracle value (fp32, un-rounded) and noise bound of out[rows, cols] for the
    [N,K] weight layout; all arguments CPU tensors, cols on 128-column boundaries."""
    a8w, asw = a8[rows], a_s[rows]
    b8w = b8_nk[cols]
    bsw = b_s_nk[cols.start // 128: -(-cols.stop // 128)]
    ref32 = orc.fp8_gemm_blockwise(a8w, b8w, asw, bsw, 128, 128, "nk", out_dtype=None)
    noise = accumulation_noise(orc.dequantize_a(a8w, asw).abs(), orc.dequantize_b(b8w, bsw, 128, 128, "nk").abs(),
                               a8.shape[1])
    return ref32, noise
