"""GPU: the quantized GEMMs through the C ABI against the oracle.

Acceptance (stated in the benchmark definition of this path): relative
Frobenius error <= 1e-3 against the fp32-accumulated oracle value and
|err| <= 2 bf16 ulp of that value per element; elements whose deviation is
within the fp32 accumulation-order noise floor are counted separately (see
_util.check_gemm)."""
import os

import pytest
import torch

import ks_oracle as orc
from _util import (accumulation_noise, block_quant_nk_device, check_gemm, fp8_inputs, fp8_window_reference,
                   from_bits16, from_u8, gen, golden, quant_group_device, w4a16_inputs)

pytestmark = pytest.mark.gpu


class fp8_path:
    """Pins the kernel choice of the FP8 GEMM for the duration of a block."""

    def __init__(self, path=None, bn=None):
        self.vals = {"KS_B200_FP8_PATH": path, "KS_B200_FP8_BN": str(bn) if bn else None}

    def __enter__(self):
        self.old = {k: os.environ.get(k) for k in self.vals}
        for k, v in self.vals.items():
            if v is None:
                os.environ.pop(k, None)
            else:
                os.environ[k] = v

    def __exit__(self, *a):
        for k, v in self.old.items():
            if v is None:
                os.environ.pop(k, None)
            else:
                os.environ[k] = v


def fp8_reference(a8, a_s, b8, b_s, bn=128, bk=128):
    ref32 = orc.fp8_gemm_blockwise(a8, b8, a_s, b_s, bn, bk, "kn", out_dtype=None)
    a_abs = orc.dequantize_a(a8, a_s, bk).abs()
    b_abs = orc.dequantize_b(b8, b_s, bn, bk).abs()
    return ref32, accumulation_noise(a_abs, b_abs, a8.shape[1])


def run_fp8(ks, dev, a8, a_s, b8_kn, b_s_kn, layout, out_dtype=torch.bfloat16, bn=128, bk=128):
    if layout == "kn":
        b, bs = b8_kn, b_s_kn
    else:
        b, bs = b8_kn.t().contiguous(), b_s_kn.t().contiguous()
    out = ks.dispatch.fp8_gemm_blockwise(a8.to(dev), b.to(dev), a_s.to(dev), bs.to(dev), block_n=bn, block_k=bk,
                                         out_dtype=out_dtype, b_layout=layout)
    torch.cuda.synchronize()
    ks.runtime.stream_synchronize(0)  # surfaces a kernel that gave up on a bounded wait
    return out.cpu()


@pytest.mark.parametrize("m,n,k,bn,bk,layout,out_dtype,fp8", [
    (40, 200, 300, 128, 128, "kn", torch.float32, "e4m3"),
    (40, 200, 300, 128, 128, "nk", torch.bfloat16, "e4m3"),
    (65, 130, 96, 64, 32, "kn", torch.float16, "e4m3"),
    (17, 64, 256, 128, 128, "kn", torch.bfloat16, "e5m2"),
    (1, 48, 128, 16, 64, "nk", torch.float32, "e4m3"),
])
def test_fp8_general_kernel(ks, cuda, m, n, k, bn, bk, layout, out_dtype, fp8):
    a8, a_s, b8, b_s = fp8_inputs(m, n, k, seed=m + n + k, block_n=bn, block_k=bk, fp8=fp8)
    ref32, noise = fp8_reference(a8, a_s, b8, b_s, bn, bk)
    with fp8_path("general"):
        out = run_fp8(ks, cuda, a8, a_s, b8, b_s, layout, out_dtype, bn, bk)
    ulps = 2.0 if out_dtype == torch.bfloat16 else 2.0  # f16/f32 outputs are tighter than 2 bf16 ulp
    check_gemm(out, ref32, noise, f"general {m}x{n}x{k} {layout}", ulps=ulps)


@pytest.mark.parametrize("m,n,k,layout,bn_tile,out_dtype,fp8", [
    (128, 128, 128, "nk", 128, torch.float32, "e4m3"),     # one tile, one K-block
    (128, 256, 256, "nk", 256, torch.float32, "e4m3"),
    (128, 128, 128, "kn", 128, torch.float32, "e4m3"),     # MN-major B operand
    (128, 256, 256, "kn", 256, torch.float32, "e4m3"),
    (256, 512, 1024, "nk", 256, torch.bfloat16, "e4m3"),
    (256, 512, 1024, "kn", 128, torch.bfloat16, "e4m3"),
    (200, 336, 400, "nk", 256, torch.bfloat16, "e4m3"),    # ragged M, N, K (K % 16 == 0)
    (200, 336, 400, "kn", 256, torch.float16, "e4m3"),
    (77, 144, 272, "kn", 128, torch.float32, "e5m2"),
    (1, 7168, 512, "nk", 128, torch.bfloat16, "e4m3"),     # decode-like single row
    (1024, 2048, 7168, "nk", 256, torch.bfloat16, "e4m3"),  # 64 tiles (one per CTA), 56 K-blocks
    (1024, 2048, 7168, "kn", 256, torch.bfloat16, "e4m3"),
    (2304, 3328, 1024, "nk", 256, torch.bfloat16, "e4m3"),  # 18 x 13 tiles: partial last panel, partial last round
    (2304, 3328, 1024, "kn", 256, torch.float32, "e4m3"),
    (2304, 3328, 1024, "nk", 128, torch.bfloat16, "e4m3"),  # 18 x 26 narrow tiles: 3.2 rounds
    (2500, 2000, 4096, "nk", 256, torch.bfloat16, "e4m3"),  # 160 tiles: 12 left for a K-split round of 8 parts,
    (2500, 2000, 4096, "kn", 256, torch.float16, "e4m3"),   # among them the ragged last row and column tiles
])
def test_fp8_tcgen05_kernel(ks, cuda, m, n, k, layout, bn_tile, out_dtype, fp8):
    a8, a_s, b8, b_s = fp8_inputs(m, n, k, seed=m * 7 + n + k, fp8=fp8)
    ref32, noise = fp8_reference(a8, a_s, b8, b_s)
    with fp8_path("tcgen05", bn_tile):
        out = run_fp8(ks, cuda, a8, a_s, b8, b_s, layout, out_dtype)
    check_gemm(out, ref32, noise, f"tcgen05 {m}x{n}x{k} {layout} bn{bn_tile}")
    # and against the general kernel on the same inputs (fp32 out: order noise only)
    if out_dtype == torch.float32:
        with fp8_path("general"):
            gen_out = run_fp8(ks, cuda, a8, a_s, b8, b_s, layout, out_dtype)
        assert orc.rel_frobenius(out, gen_out) < 1e-5



def _headline_inputs(m, n, k, dev, seed):
    """Operands of a BASELINE-sized dense problem, made on the device (weights ~N(0, 0.02)
    block-quantized 128 x 128, activations ~N(0,1) quantized 1 x 128), [N,K] layout."""
    g = torch.Generator(device=dev).manual_seed(seed)
    a = torch.randn(m, k, generator=g, device=dev).to(torch.bfloat16)
    a8, a_s = quant_group_device(a)
    b8, b_s = block_quant_nk_device(torch.randn(n, k, generator=g, device=dev) * 0.02)
    return a8, a_s, b8, b_s


@pytest.mark.parametrize("m,n,k,layout,windows", [
    # the benchmark's headline problem: 32 x 28 = 896 tiles on 148 CTAs (6.05 rounds)
    (4096, 7168, 7168, "nk", [(0, 0), (3584, 6144), (1792, 3072)]),
    (4096, 7168, 7168, "kn", [(3584, 6144), (512, 1024)]),
    # one K-shard of the row-parallel configuration at 8 GPUs
    (16384, 8192, 3584, "nk", [(0, 0), (15872, 7168)]),
])
def test_fp8_baseline_shapes(ks, cuda, m, n, k, layout, windows):
    """The full-size problems, default kernel choice. The oracle checks 512 x 1024 windows
    element by element; the general kernel (the reference kernel's summation order) checks
    every element of the output on the device."""
    a8, a_s, b8, b_s = _headline_inputs(m, n, k, cuda, seed=m + n + k)
    if layout == "kn":
        b_run, bs_run = b8.t().contiguous(), b_s.t().contiguous()
    else:
        b_run, bs_run = b8, b_s
    out = ks.dispatch.fp8_gemm_blockwise(a8, b_run, a_s, bs_run, b_layout=layout)
    torch.cuda.synchronize()
    ks.runtime.stream_synchronize(0)
    a8c, asc, b8c, bsc = a8.cpu(), a_s.cpu(), b8.cpu(), b_s.cpu()
    for (r0, c0) in windows:
        rows, cols = slice(r0, r0 + 512), slice(c0, c0 + 1024)
        ref32, noise = fp8_window_reference(a8c, asc, b8c, bsc, rows, cols)
        check_gemm(out[rows, cols].cpu(), ref32, noise, f"{m}x{n}x{k} {layout} window ({r0},{c0})")
    with fp8_path("general"):
        full = ks.dispatch.fp8_gemm_blockwise(a8, b_run, a_s, bs_run, b_layout=layout, out_dtype=torch.float32)
        torch.cuda.synchronize()
    diff = (out.float() - full).double()
    frob = float(diff.norm() / full.double().norm())
    assert frob < 3e-3, f"whole output vs general kernel: {frob}"
    # nothing worse than bf16 rounding of a correct value anywhere (a wrong tile would be O(1) off)
    worst = float((diff.abs() / (full.abs().double() + 1e-2 * float(full.abs().max()))).max())
    assert worst < 0.02, f"worst element vs general kernel: {worst}"


def test_fp8_golden(ks, cuda):
    for tag in ("a", "b"):
        g = golden(f"fp8_blockwise_{tag}.npz")
        a8 = from_u8(g["a8"], torch.float8_e4m3fn)
        b8 = from_u8(g["b8"], torch.float8_e4m3fn)
        a_s, b_s = torch.from_numpy(g["a_scale"]), torch.from_numpy(g["b_scale"])
        ref = torch.from_numpy(g["ref"])
        for layout in ("kn", "nk"):
            out = run_fp8(ks, cuda, a8, a_s, b8, b_s, layout, torch.float32)
            assert orc.rel_frobenius(out, ref) < 1e-5, (tag, layout)
            out16 = run_fp8(ks, cuda, a8, a_s, b8, b_s, layout, torch.bfloat16)
            _, noise = fp8_reference(a8, a_s, b8, b_s)
            check_gemm(out16, ref, noise, f"golden {tag} {layout}")


@pytest.mark.parametrize("m,k,n,gs,dtype,zeros,bias", [
    (16, 4096, 4096, 128, torch.bfloat16, True, False),   # the CPU-runnable configuration
    (1, 256, 192, 128, torch.bfloat16, True, False),
    (5, 128, 72, 32, torch.float16, True, True),
    (33, 512, 100, 64, torch.bfloat16, False, True),      # zeros == NULL means zero-point 0
    (8, 256, 64, -1, torch.float16, True, False),         # group_size <= 0: one group over K
    (130, 384, 136, 128, torch.bfloat16, True, False),
])
def test_w4a16(ks, cuda, m, k, n, gs, dtype, zeros, bias):
    a, codes, scales, zp = w4a16_inputs(m, k, n, gs, dtype, seed=m + k + n, with_zeros=zeros)
    b_packed = orc.pack_int4_bytes(codes)
    bias_t = torch.randn(n, generator=gen(5)).to(dtype) if bias else None
    ref32 = orc.w4a16(a, b_packed, scales, zp, gs, bias_t, out_dtype=None)
    w = orc.w4a16_weight(b_packed, scales, zp, gs).float()
    noise = accumulation_noise(a.float().abs(), w.abs(), k)
    out = ks.dispatch.w4a16(a.to(cuda), b_packed.to(cuda), scales.to(cuda), zp.to(cuda) if zp is not None else None,
                            group_size=gs, bias=bias_t.to(cuda) if bias else None)
    torch.cuda.synchronize()
    assert out.dtype == dtype and out.shape == (m, n)
    check_gemm(out.cpu(), ref32, noise, f"w4a16 {m}x{n}x{k}")


class w4_path:
    def __init__(self, path):
        self.path = path

    def __enter__(self):
        self.old = os.environ.get("KS_B200_W4A16_PATH")
        os.environ["KS_B200_W4A16_PATH"] = self.path

    def __exit__(self, *a):
        if self.old is None:
            os.environ.pop("KS_B200_W4A16_PATH", None)
        else:
            os.environ["KS_B200_W4A16_PATH"] = self.old


@pytest.mark.parametrize("m,k,n,gs,dtype,zeros,bias", [
    (1, 128, 128, 128, torch.bfloat16, "eight", False),      # one unit
    (16, 256, 128, 128, torch.bfloat16, "eight", False),
    (16, 128, 256, 128, torch.bfloat16, "eight", False),
    (8, 4096, 256, 128, torch.bfloat16, "eight", True),      # each column tile split over 32 CTAs
    (32, 1024, 2048, 128, torch.bfloat16, "random", False),  # integer zero-points 0..15
    (32, 1024, 2048, 256, torch.float16, "random", True),    # two K-steps per scale group
    (5, 512, 208, 128, torch.bfloat16, None, False),         # ragged last column tile, zeros == NULL
    (128, 512, 384, 128, torch.bfloat16, "eight", False),    # full token tile
    (77, 384, 512, 128, torch.float16, "fraction", False),   # non-integer zero-points: exact fp32 path
    (300, 256, 640, 128, torch.bfloat16, "eight", True),     # several token tiles
    (32, 4096, 28672 // 8, 128, torch.bfloat16, "eight", False),
    (4, 4096, 14336, 128, torch.bfloat16, "random", False),   # ~24 units per CTA: every ring wraps several times
    (16, 7168, 4608, 128, torch.float16, "eight", True),      # 56 K-steps per column tile, ~14 units per CTA
])
def test_w4a16_tcgen05(ks, cuda, m, k, n, gs, dtype, zeros, bias):
    g = gen(m + k + n)
    a = torch.randn(m, k, generator=g).to(dtype)
    codes = torch.randint(0, 16, (k, n), generator=g).to(torch.int32)
    scales = (torch.randn(k // gs, n, generator=g).mul(0.02).abs() + 1e-3).to(dtype)
    if zeros == "eight":
        zp = torch.full((k // gs, n), 8.0).to(dtype)
    elif zeros == "random":
        zp = torch.randint(0, 16, (k // gs, n), generator=g).to(dtype)
    elif zeros == "fraction":
        zp = (torch.rand(k // gs, n, generator=g) * 15).to(dtype)
    else:
        zp = None
    b_packed = orc.pack_int4_bytes(codes)
    bias_t = torch.randn(n, generator=g).to(dtype) if bias else None
    ref32 = orc.w4a16(a, b_packed, scales, zp, gs, bias_t, out_dtype=None)
    w = orc.w4a16_weight(b_packed, scales, zp, gs).float()
    noise = accumulation_noise(a.float().abs(), w.abs(), k)
    with w4_path("tcgen05"):
        out = ks.dispatch.w4a16(a.to(cuda), b_packed.to(cuda), scales.to(cuda),
                                zp.to(cuda) if zp is not None else None, group_size=gs,
                                bias=bias_t.to(cuda) if bias else None)
        torch.cuda.synchronize()
        ks.runtime.stream_synchronize(0)
        # a second call reuses the scratch memory (counters must have reset themselves)
        out2 = ks.dispatch.w4a16(a.to(cuda), b_packed.to(cuda), scales.to(cuda),
                                 zp.to(cuda) if zp is not None else None, group_size=gs,
                                 bias=bias_t.to(cuda) if bias else None)
        torch.cuda.synchronize()
    check_gemm(out.cpu(), ref32, noise, f"w4a16 tcgen05 {m}x{n}x{k}")
    assert torch.equal(out.cpu().view(torch.int16), out2.cpu().view(torch.int16)), "not reproducible run to run"
    with w4_path("general"):
        gen_out = ks.dispatch.w4a16(a.to(cuda), b_packed.to(cuda), scales.to(cuda),
                                    zp.to(cuda) if zp is not None else None, group_size=gs,
                                    bias=bias_t.to(cuda) if bias else None)
        torch.cuda.synchronize()
    # both kernels multiply the same rounded weights; they differ by summation order only
    assert orc.rel_frobenius(out.cpu().float(), gen_out.cpu().float()) < 2e-3



@pytest.mark.parametrize("m,k,n,gs,dtype,zeros,bias", [
    (1, 128, 256, 128, torch.bfloat16, "eight", False),       # one unit
    (8, 256, 256, 128, torch.bfloat16, "eight", False),
    (16, 128, 512, 128, torch.bfloat16, "eight", False),
    (8, 4096, 256, 128, torch.bfloat16, "eight", True),       # one column tile split over 32 CTAs
    (32, 1024, 2048, 128, torch.bfloat16, "random", False),   # integer zero-points 0..15
    (32, 1024, 2048, 256, torch.float16, "random", True),     # two K-steps per scale group
    (5, 512, 208, 128, torch.bfloat16, None, False),          # ragged last column tile, zeros == NULL
    (64, 512, 384, 128, torch.bfloat16, "eight", False),      # the widest token tile
    (41, 384, 512, 128, torch.float16, "fraction", False),    # non-integer zero-points: exact fp32 path
    (9, 640, 1040, 640, torch.bfloat16, "eight", True),       # one group over K, two token groups, ragged N
    (32, 4096, 28672 // 8, 128, torch.bfloat16, "eight", False),
    (4, 4096, 14336, 128, torch.bfloat16, "random", False),   # ~12 units per CTA: the ring wraps
    (16, 7168, 4608, 128, torch.float16, "eight", True),      # 56 K-steps per column tile
])
def test_w4a16_decode_kernel(ks, cuda, m, k, n, gs, dtype, zeros, bias):
    """The register-operand decode kernel against the oracle, twice in a row (the second call
    finds the split-K counters as the first left them) and against the general kernel."""
    g = gen(m + k + n)
    a = torch.randn(m, k, generator=g).to(dtype)
    codes = torch.randint(0, 16, (k, n), generator=g).to(torch.int32)
    scales = (torch.randn(k // gs, n, generator=g).mul(0.02).abs() + 1e-3).to(dtype)
    zp = {"eight": lambda: torch.full((k // gs, n), 8.0).to(dtype),
          "random": lambda: torch.randint(0, 16, (k // gs, n), generator=g).to(dtype),
          "fraction": lambda: (torch.rand(k // gs, n, generator=g) * 15).to(dtype),
          None: lambda: None}[zeros]()
    b_packed = orc.pack_int4_bytes(codes)
    bias_t = torch.randn(n, generator=g).to(dtype) if bias else None
    ref32 = orc.w4a16(a, b_packed, scales, zp, gs, bias_t, out_dtype=None)
    w = orc.w4a16_weight(b_packed, scales, zp, gs).float()
    noise = accumulation_noise(a.float().abs(), w.abs(), k)
    args = (a.to(cuda), b_packed.to(cuda), scales.to(cuda), zp.to(cuda) if zp is not None else None)
    kw = dict(group_size=gs, bias=bias_t.to(cuda) if bias else None)
    with w4_path("decode"):
        out = ks.dispatch.w4a16(*args, **kw)
        out2 = ks.dispatch.w4a16(*args, **kw)
        torch.cuda.synchronize()
        ks.runtime.stream_synchronize(0)
    check_gemm(out.cpu(), ref32, noise, f"w4a16 decode {m}x{n}x{k}")
    assert torch.equal(out.cpu().view(torch.int16), out2.cpu().view(torch.int16)), "not reproducible run to run"
    with w4_path("general"):
        gen_out = ks.dispatch.w4a16(*args, **kw)
        torch.cuda.synchronize()
    assert orc.rel_frobenius(out.cpu().float(), gen_out.cpu().float()) < 2e-3


@pytest.mark.parametrize("path", ["decode", "tcgen05"])
def test_w4a16_recovers_from_dirty_split_counters(ks, cuda, path):
    """A launch that gives up on a bounded wait can leave split-K arrival counters non-zero; the
    fault poll marks every stream's counters and the next call clears them. Staged here without
    any GPU fault: a test hook fills the counters with garbage and sets the same mark."""
    m, k, n, gs = 8, 4096, 512, 128           # every column tile is shared by several CTAs
    g = gen(77)
    a = torch.randn(m, k, generator=g).to(torch.bfloat16)
    codes = torch.randint(0, 16, (k, n), generator=g).to(torch.int32)
    scales = (torch.randn(k // gs, n, generator=g).mul(0.02).abs() + 1e-3).to(torch.bfloat16)
    zp = torch.full((k // gs, n), 8.0).to(torch.bfloat16)
    b_packed = orc.pack_int4_bytes(codes)
    args = (a.to(cuda), b_packed.to(cuda), scales.to(cuda), zp.to(cuda))
    with w4_path(path):
        clean = ks.dispatch.w4a16(*args, group_size=gs)
        torch.cuda.synchronize()
        os.environ["KS_B200_TEST_DIRTY_COUNTERS"] = "1"
        try:
            after = ks.dispatch.w4a16(*args, group_size=gs)
            torch.cuda.synchronize()
        finally:
            os.environ.pop("KS_B200_TEST_DIRTY_COUNTERS", None)
        again = ks.dispatch.w4a16(*args, group_size=gs)
        torch.cuda.synchronize()
        ks.runtime.stream_synchronize(0)
    assert torch.equal(clean, after) and torch.equal(clean, again)
    ref32 = orc.w4a16(a, b_packed, scales, zp, gs, None, out_dtype=None)
    assert orc.rel_frobenius(clean.cpu().float(), ref32) < 3e-3


@pytest.mark.parametrize("k,n", [(4096, 28672), (14336, 4096)])
def test_w4a16_baseline_shapes(ks, cuda, k, n):
    """The decode sweep of the benchmark (Llama-3-8B MLP shapes, M in {1, 8, 32, 128}), default
    kernel choice; the oracle checks three windows of 1024 columns (first, middle, last)."""
    g = gen(k + n)
    codes_b = torch.randint(0, 256, (k // 2, n), generator=g, dtype=torch.uint8)     # code = q + 8, q uniform
    scales = (torch.randn(k // 128, n, generator=g).mul(0.02).abs() + 1e-3).to(torch.bfloat16)
    zeros = torch.full((k // 128, n), 8.0).to(torch.bfloat16)
    bp_d, sc_d, zp_d = codes_b.to(cuda), scales.to(cuda), zeros.to(cuda)
    windows = [slice(0, 1024), slice(n // 2 - 256, n // 2 + 768), slice(n - 1024, n)]
    wref = [(orc.w4a16_weight(codes_b[:, w], scales[:, w], zeros[:, w], 128).float()) for w in windows]
    for m in (1, 8, 32, 128):
        a = torch.randn(m, k, generator=g).to(torch.bfloat16)
        out = ks.dispatch.w4a16(a.to(cuda), bp_d, sc_d, zp_d, group_size=128)
        torch.cuda.synchronize()
        ks.runtime.stream_synchronize(0)
        out = out.cpu()
        for w, wf in zip(windows, wref):
            ref32 = a.float() @ wf
            noise = accumulation_noise(a.float().abs(), wf.abs(), k)
            check_gemm(out[:, w], ref32, noise, f"w4a16 M={m} K={k} N={n} columns {w.start}..{w.stop}")


@pytest.mark.parametrize("operand", ["smem", "tmem"])
@pytest.mark.parametrize("m,k,n,gs,dtype,zeros", [
    (8, 1024, 512, 128, torch.bfloat16, "random"),
    (32, 512, 208, 256, torch.float16, "eight"),      # ragged last column tile, two K-steps per group
    (3, 768, 128, 128, torch.bfloat16, "fraction"),   # K = 6 steps, fp32 fallback for the zero-points
    (17, 256, 384, 128, torch.bfloat16, None),
])
def test_w4a16_operand_paths(ks, cuda, operand, m, k, n, gs, dtype, zeros):
    """Decode shapes through both ways of feeding the tensor core (shared-memory operand,
    tensor-memory operand); both multiply the same rounded weights and differ by the
    order of the fp32 sums only."""
    g = gen(m * 3 + k + n)
    a = torch.randn(m, k, generator=g).to(dtype)
    codes = torch.randint(0, 16, (k, n), generator=g).to(torch.int32)
    scales = (torch.randn(k // gs, n, generator=g).mul(0.02).abs() + 1e-3).to(dtype)
    zp = {"eight": lambda: torch.full((k // gs, n), 8.0).to(dtype),
          "random": lambda: torch.randint(0, 16, (k // gs, n), generator=g).to(dtype),
          "fraction": lambda: (torch.rand(k // gs, n, generator=g) * 15).to(dtype),
          None: lambda: None}[zeros]()
    b_packed = orc.pack_int4_bytes(codes)
    ref32 = orc.w4a16(a, b_packed, scales, zp, gs, None, out_dtype=None)
    noise = accumulation_noise(a.float().abs(), orc.w4a16_weight(b_packed, scales, zp, gs).float().abs(), k)
    old = os.environ.get("KS_B200_W4A16_OPERAND")
    outs = {}
    try:
        for path in ("smem", "tmem"):
            os.environ["KS_B200_W4A16_OPERAND"] = path
            with w4_path("tcgen05"):
                outs[path] = ks.dispatch.w4a16(a.to(cuda), b_packed.to(cuda), scales.to(cuda),
                                               zp.to(cuda) if zp is not None else None, group_size=gs).cpu()
            torch.cuda.synchronize()
            ks.runtime.stream_synchronize(0)
    finally:
        if old is None:
            os.environ.pop("KS_B200_W4A16_OPERAND", None)
        else:
            os.environ["KS_B200_W4A16_OPERAND"] = old
    check_gemm(outs[operand], ref32, noise, f"w4a16 {operand} operand {m}x{n}x{k}")
    assert orc.rel_frobenius(outs["smem"].float(), outs["tmem"].float()) < 2e-3


def test_w4a16_scratch_survives_shape_changes(ks, cuda):
    """Split-K bookkeeping must not depend on what an earlier shape left in the library's
    scratch memory: a problem with few column tiles (its partial sums land low in the
    scratch) followed by one with many column tiles (whose arrival counters must all start
    at zero), twice over."""
    g = gen(4242)
    cases = []
    for (m, k, n) in ((8, 4096, 256), (4, 4096, 14336), (16, 2048, 384), (4, 4096, 14336)):
        a = torch.randn(m, k, generator=g).to(torch.bfloat16)
        codes = torch.randint(0, 16, (k, n), generator=g).to(torch.int32)
        scales = (torch.randn(k // 128, n, generator=g).mul(0.02).abs() + 1e-3).to(torch.bfloat16)
        zp = torch.randint(0, 16, (k // 128, n), generator=g).to(torch.bfloat16)
        bp = orc.pack_int4_bytes(codes)
        cases.append((m, k, n, a, bp, scales, zp))
    with w4_path("tcgen05"):
        outs = [ks.dispatch.w4a16(a.to(cuda), bp.to(cuda), sc.to(cuda), zp.to(cuda), group_size=128)
                for (_, _, _, a, bp, sc, zp) in cases]
        torch.cuda.synchronize()
        ks.runtime.stream_synchronize(0)
    for (m, k, n, a, bp, sc, zp), out in zip(cases, outs):
        ref32 = orc.w4a16(a, bp, sc, zp, 128, None, out_dtype=None)
        noise = accumulation_noise(a.float().abs(), orc.w4a16_weight(bp, sc, zp, 128).float().abs(), k)
        check_gemm(out.cpu(), ref32, noise, f"w4a16 in sequence {m}x{n}x{k}")


def test_w4a16_golden(ks, cuda):
    for tag, dt in (("bf16", torch.bfloat16), ("f16", torch.float16)):
        g = golden(f"w4a16_{tag}.npz")
        a = from_bits16(g["a"], dt)
        bp = torch.from_numpy(g["b_packed"])
        sc, zp = from_bits16(g["scales"], dt), from_bits16(g["zeros"], dt)
        gs = int(g["group_size"])
        out = ks.dispatch.w4a16(a.to(cuda), bp.to(cuda), sc.to(cuda), zp.to(cuda), group_size=gs).cpu()
        ref = from_bits16(g["out"], dt).float()
        ref32 = orc.w4a16(a, bp, sc, zp, gs, out_dtype=None)
        # the frozen output is the rounded reference; ours may differ from it by one rounding step
        check_gemm(out, ref32, accumulation_noise(a.float().abs(), orc.w4a16_weight(bp, sc, zp, gs).float().abs(),
                                                  a.shape[1]), f"w4a16 golden {tag}")
        assert orc.rel_frobenius(out.float(), ref) < 2e-3


def ragged_offsets(rows_per_expert):
    off = [0]
    for r in rows_per_expert:
        off.append(off[-1] + r)
    return torch.tensor(off, dtype=torch.int32)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_grouped_gemm_plain(ks, cuda, dtype):
    offs = ragged_offsets([5, 0, 70, 1, 64, 0])
    total, k, n, e = int(offs[-1]), 96, 80, 6
    g = gen(9)
    a = torch.randn(total, k, generator=g).to(dtype)
    b = torch.randn(e, k, n, generator=g).to(dtype)
    out = ks.dispatch.moe(a.to(cuda), b.to(cuda), offs.to(cuda), num_experts=e, n=n, k=k)
    torch.cuda.synchronize()
    ref32 = orc.grouped_gemm(a, b, offs.tolist(), out_dtype=None)
    assert orc.rel_frobenius(out.cpu().float(), ref32) < (1e-6 if dtype == torch.float32 else 3e-3)
    if dtype == torch.bfloat16:
        g2 = golden("grouped_gemm_bf16.npz")
        a2, b2 = from_bits16(g2["a"], dtype), from_bits16(g2["b"], dtype)
        o2 = torch.from_numpy(g2["offsets"])
        out2 = ks.dispatch.moe(a2.to(cuda), b2.to(cuda), o2.to(cuda), num_experts=b2.shape[0], n=b2.shape[2],
                               k=b2.shape[1]).cpu()
        assert orc.rel_frobenius(out2.float(), from_bits16(g2["out"], dtype).float()) < 3e-3


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("rows,n,k", [
    ([130, 0, 257, 1, 128, 64, 0, 300], 512, 1024),     # ragged experts, several row tiles each
    ([17, 200, 3], 264, 200),                            # N and K with partial tiles (multiples of 8 only)
    ([128] * 32, 2048, 768),                             # more tiles than SMs
    ([200] * 24 + [520, 129], 2048, 512),                # several row tiles per expert
])
def test_grouped_gemm_plain_tensor_core(ks, cuda, dtype, rows, n, k):
    """f16 / bf16 grouped GEMM on the tcgen05 mainloop (16-bit mode) against the oracle with the
    usual GEMM bound, and against the SIMT kernel."""
    offs = ragged_offsets(rows)
    total, e = int(offs[-1]), len(rows)
    g = gen(total + n + k)
    a = torch.randn(total, k, generator=g).to(dtype)
    b = (torch.randn(e, k, n, generator=g) * 0.05).to(dtype)
    args = (a.to(cuda), b.to(cuda), offs.to(cuda))
    out = ks.dispatch.moe(*args, num_experts=e, n=n, k=k)
    out2 = ks.dispatch.moe(*args, num_experts=e, n=n, k=k)
    torch.cuda.synchronize()
    ks.runtime.stream_synchronize(0)
    ref32 = orc.grouped_gemm(a, b, offs.tolist(), out_dtype=None)
    noise = torch.zeros_like(ref32)
    for i in range(e):
        lo, hi = int(offs[i]), int(offs[i + 1])
        if hi > lo:
            noise[lo:hi] = accumulation_noise(a[lo:hi].float().abs(), b[i].float().abs(), k)
    if dtype == torch.bfloat16:
        check_gemm(out.cpu(), ref32, noise, f"grouped {dtype} {total}x{n}x{k}")
    assert orc.rel_frobenius(out.cpu().float(), ref32) < 3e-3
    assert torch.equal(out, out2)
    old = os.environ.get("KS_B200_GROUPED_PATH")
    os.environ["KS_B200_GROUPED_PATH"] = "general"
    try:
        simt = ks.dispatch.moe(*args, num_experts=e, n=n, k=k)
        torch.cuda.synchronize()
    finally:
        if old is None:
            os.environ.pop("KS_B200_GROUPED_PATH", None)
        else:
            os.environ["KS_B200_GROUPED_PATH"] = old
    assert orc.rel_frobenius(out.cpu().float(), simt.cpu().float()) < 3e-3


def test_grouped_gemm_plain_fp8_operands(ks, cuda):
    """fp8 dtype: raw code values multiplied, C written in the same fp8 type."""
    offs = ragged_offsets([3, 20])
    g = gen(4)
    a = torch.randn(23, 32, generator=g).to(torch.float8_e4m3fn)
    b = (torch.randn(2, 32, 16, generator=g) * 0.5).to(torch.float8_e4m3fn)
    out = ks.dispatch.moe(a.to(cuda), b.to(cuda), offs.to(cuda), num_experts=2, n=16, k=32).cpu()
    ref = orc.grouped_gemm(a, b, offs.tolist(), out_dtype=None).clamp(-448, 448).to(torch.float8_e4m3fn)
    assert (out.float() - ref.float()).abs().max() <= 0.13 * ref.float().abs().max()


@pytest.mark.parametrize("layout,path,n,k", [
    ("nk", "general", 200, 300),
    ("kn", "general", 200, 300),
    ("nk", "tcgen05", 512, 384),
    ("kn", "tcgen05", 512, 384),
    ("nk", "tcgen05", 336, 400),
    ("nk", "tcgen05", 200, 1040),
])
def test_grouped_gemm_fp8_blockwise(ks, cuda, layout, path, n, k):
    rows = [130, 0, 7, 256, 1, 129, 0, 64, 300, 16, 17, 513]
    e = len(rows)
    offs = ragged_offsets(rows)
    total = int(offs[-1])
    g = gen(n + k)
    a = torch.randn(total, k, generator=g).to(torch.bfloat16)
    a8, a_s = orc.quantize_fp8_group(a, 128)
    b8_l, bs_l = [], []
    for _ in range(e):
        w_kn = torch.randn(k, n, generator=g) * 0.02
        b8, bs = orc.quantize_weight_blocks(w_kn, 128, 128)
        if layout == "nk":
            b8, bs = b8.t().contiguous(), bs.t().contiguous()
        b8_l.append(b8)
        bs_l.append(bs)
    b8, bs = torch.stack(b8_l), torch.stack(bs_l)
    ref32 = orc.grouped_gemm_fp8_blockwise(a8, b8, a_s, bs, offs.tolist(), layout=layout, out_dtype=None)
    with fp8_path(path):
        out = ks.dispatch.moe(a8.to(cuda), b8.to(cuda), offs.to(cuda), num_experts=e, n=n, k=k, a_scale=a_s.to(cuda),
                              b_scale=bs.to(cuda), b_layout=layout)
        torch.cuda.synchronize()
        ks.runtime.stream_synchronize(0)
    noise = torch.full_like(ref32, float(ref32.abs().max()) * 1e-5)
    check_gemm(out.cpu(), ref32, noise, f"grouped fp8 {layout} {path}")


@pytest.mark.parametrize("n,k", [(4096, 7168), (7168, 2048)])
def test_grouped_gemm_fp8_256_experts(ks, cuda, n, k):
    """The MoE configuration's expert count and GEMM sizes: 256 experts, rows per expert from a
    top-8 routing of 4096 tokens (ragged), experts 3 and 200 emptied. The oracle checks the rows
    of four experts; weights are made on the device, one expert at a time."""
    e = 256
    gr = gen(17)
    _, ids = orc.moe_route(torch.randn(4096, e, generator=gr), 8)
    counts = torch.bincount(ids.reshape(-1), minlength=e)
    counts[3] = 0
    counts[200] = 0
    offs = torch.zeros(e + 1, dtype=torch.int32)
    offs[1:] = torch.cumsum(counts, 0).to(torch.int32)
    total = int(offs[-1])
    gd = torch.Generator(device=cuda).manual_seed(n + k)
    a = torch.randn(total, k, generator=gd, device=cuda).to(torch.bfloat16)
    a8, a_s = quant_group_device(a)
    b8 = torch.empty(e, n, k, dtype=torch.float8_e4m3fn, device=cuda)
    b_s = torch.empty(e, n // 128, k // 128, dtype=torch.float32, device=cuda)
    for i in range(e):
        b8[i], b_s[i] = block_quant_nk_device(torch.randn(n, k, generator=gd, device=cuda) * 0.02)
    out = ks.dispatch.moe(a8, b8, offs.to(cuda), num_experts=e, n=n, k=k, a_scale=a_s, b_scale=b_s, b_layout="nk")
    torch.cuda.synchronize()
    ks.runtime.stream_synchronize(0)
    biggest = int(torch.argmax(counts))
    for i in (0, 2, biggest, e - 1):
        lo, hi = int(offs[i]), int(offs[i + 1])
        if hi == lo:
            continue
        a8c, asc, b8c, bsc = a8[lo:hi].cpu(), a_s[lo:hi].cpu(), b8[i].cpu(), b_s[i].cpu()
        ref32 = orc.fp8_gemm_blockwise(a8c, b8c, asc, bsc, 128, 128, "nk", out_dtype=None)
        noise = accumulation_noise(orc.dequantize_a(a8c, asc).abs(), orc.dequantize_b(b8c, bsc, 128, 128, "nk").abs(), k)
        check_gemm(out[lo:hi].cpu(), ref32, noise, f"256 experts, expert {i} ({hi - lo} rows) n={n} k={k}")
    # rows of the emptied experts do not exist; the row after them belongs to the next expert
    assert int(offs[4]) == int(offs[3]) and int(offs[201]) == int(offs[200])
