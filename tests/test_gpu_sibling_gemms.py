"""GPU: the GEMMs that share the FP8 mainloop (ks_gemm_fp8 with per-token / per-channel
scales, ks_gemm_w8a8 on kind::i8, the masked grouped layout) through the C ABI against the
oracle's restatement of the reference's arithmetic (kernels/src/gemm/gemm_fp8.cu:147-153,
gemm_w8a8.cu:134-141 with benchmarks/bench.py:1228-1232).

Bars: int8 accumulation is exact, so ks_gemm_w8a8 with an fp32 output must equal the oracle
bit for bit; 16-bit outputs within one rounding of the fp32 value; the FP8 GEMM within the
acceptance of the block-scaled one (relative Frobenius <= 1e-3, 2 bf16 ulp above the
accumulation-order noise floor)."""
import pytest
import torch

import ks_oracle as orc
from _util import accumulation_noise, check_gemm, gen

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("m,n,k,a_mode,b_mode,out_dtype,fp8", [
    (128, 256, 128, "token", "channel", torch.float32, "e4m3"),     # one tile, one K-block
    (300, 400, 528, "token", "channel", torch.bfloat16, "e4m3"),    # ragged M and N, K % 128 != 0
    (64, 128, 4096, "tensor", "tensor", torch.float16, "e4m3"),
    (2304, 3328, 1024, "token", "channel", torch.bfloat16, "e4m3"), # several rounds, both accumulator buffers
    (77, 144, 272, "token", "tensor", torch.float32, "e5m2"),
    (33, 50, 70, "token", "channel", torch.bfloat16, "e4m3"),       # general kernel (N % 16 != 0)
])
def test_gemm_fp8_per_token_per_channel(ks, cuda, m, n, k, a_mode, b_mode, out_dtype, fp8):
    g = gen(m + n + k)
    dt = orc.FP8_DTYPES[fp8]
    a8 = (torch.randn(m, k, generator=g) * 2).to(dt)
    b8 = (torch.randn(k, n, generator=g) * 2).to(dt)
    a_s = torch.rand(m if a_mode == "token" else 1, generator=g) * 0.02 + 0.01
    b_s = torch.rand(n if b_mode == "channel" else 1, generator=g) * 0.02 + 0.01
    out = torch.empty(m, n, dtype=out_dtype, device=cuda)
    ks.gemm.gemm_fp8(out, a8.to(cuda), b8.to(cuda), a_s.to(cuda), b_s.to(cuda), m, n, k,
                     a_mode=ks.enums.QuantMode.PER_TOKEN if a_mode == "token" else ks.enums.QuantMode.PER_TENSOR,
                     b_mode=ks.enums.QuantMode.PER_CHANNEL if b_mode == "channel" else ks.enums.QuantMode.PER_TENSOR)
    torch.cuda.synchronize()
    ks.runtime.stream_synchronize(0)
    ref32 = orc.gemm_fp8_scaled(a8, b8, a_s, b_s, out_dtype=None)
    noise = accumulation_noise(a8.float().abs() * a_s.reshape(-1, 1), b8.float().abs() * b_s.reshape(1, -1), k)
    check_gemm(out.cpu(), ref32, noise, f"gemm_fp8 {m}x{n}x{k}")


@pytest.mark.parametrize("m,n,k,a_mode,b_mode,out_dtype,bias", [
    (128, 256, 128, "token", "channel", torch.float32, False),
    (300, 400, 528, "token", "channel", torch.float32, True),
    (2304, 3328, 1024, "token", "channel", torch.bfloat16, True),
    (64, 128, 8192, "tensor", "tensor", torch.float32, False),      # |sum| far beyond 2^24: int32 must be exact
    (40, 72, 96, "token", "channel", torch.float16, True),          # general kernel (N % 16 != 0)
])
def test_gemm_w8a8(ks, cuda, m, n, k, a_mode, b_mode, out_dtype, bias):
    g = gen(m * 3 + n + k)
    a = torch.randint(-127, 127, (m, k), generator=g, dtype=torch.int8)
    b = torch.randint(-127, 127, (k, n), generator=g, dtype=torch.int8)
    if k == 8192:
        a.fill_(127)
        b.fill_(-127)           # every product -16129: the sum -1.3e8 is not an fp32 integer step away from exact
        b[::3] = 126
    a_s = torch.rand(m if a_mode == "token" else 1, generator=g) * 0.02 + 0.01
    b_s = torch.rand(n if b_mode == "channel" else 1, generator=g) * 0.02 + 0.01
    bias_t = torch.randn(n, generator=g).to(out_dtype) if bias else None
    out = torch.empty(m, n, dtype=out_dtype, device=cuda)
    ks.gemm.gemm_w8a8(out, a.to(cuda), b.to(cuda), a_s.to(cuda), b_s.to(cuda), m, n, k,
                      bias=bias_t.to(cuda) if bias else None,
                      a_mode=ks.enums.QuantMode.PER_TOKEN if a_mode == "token" else ks.enums.QuantMode.PER_TENSOR,
                      b_mode=ks.enums.QuantMode.PER_CHANNEL if b_mode == "channel" else ks.enums.QuantMode.PER_TENSOR)
    torch.cuda.synchronize()
    ks.runtime.stream_synchronize(0)
    ref32 = orc.gemm_w8a8(a, b, a_s, b_s, bias_t, out_dtype=None)
    got = out.cpu()
    if out_dtype == torch.float32:
        assert torch.equal(got, ref32), f"max diff {(got - ref32).abs().max()}"
    else:
        assert torch.equal(got, ref32.to(out_dtype)) or orc.rel_frobenius(got.float(), ref32) < 3e-3
        assert float(((got.float() - ref32).abs() / (ref32.abs() + 1e-3)).max()) < (9e-3 if out_dtype == torch.bfloat16 else 1.2e-3)


@pytest.mark.parametrize("layout,n,k,max_m", [("nk", 512, 384, 256), ("kn", 256, 512, 130), ("nk", 7168, 2048, 128)])
def test_grouped_gemm_fp8_masked_layout(ks, cuda, layout, n, k, max_m):
    """Every expert owns max_m rows and computes its first masked_m[e]; rows beyond stay
    untouched (the output is pre-filled with a marker)."""
    e = 6
    masked = torch.tensor([max_m, 0, 1, 77, max_m - 1, 128], dtype=torch.int32).clamp(max=max_m)
    g = gen(n + k + max_m)
    a = torch.randn(e, max_m, k, generator=g).to(torch.bfloat16)
    a8, a_s = orc.quantize_fp8_group(a.view(e * max_m, k), 128)
    b8_l, bs_l = [], []
    for _ in range(e):
        q, s = orc.quantize_weight_blocks(torch.randn(k, n, generator=g) * 0.02, 128, 128)
        if layout == "nk":
            q, s = q.t().contiguous(), s.t().contiguous()
        b8_l.append(q)
        bs_l.append(s)
    b8, bs = torch.stack(b8_l), torch.stack(bs_l)
    marker = 12345.0
    out = ks.dispatch.moe(a8.view(e, max_m, k).to(cuda), b8.to(cuda), n=n, k=k, a_scale=a_s.view(e, max_m, -1).to(cuda),
                          b_scale=bs.to(cuda), b_layout=layout, masked_m=masked.to(cuda),
                          out_dtype=torch.bfloat16)
    out2 = torch.full((e, max_m, n), marker, dtype=torch.bfloat16, device=cuda)
    ks.moe.grouped_gemm_fp8_blockwise_masked(out2, a8.view(e, max_m, k).to(cuda), b8.to(cuda),
                                             a_s.view(e, max_m, -1).to(cuda), bs.to(cuda), masked.to(cuda), e, max_m,
                                             n, k, b_layout=layout)
    torch.cuda.synchronize()
    ks.runtime.stream_synchronize(0)
    out, out2 = out.cpu(), out2.cpu()
    for i in range(e):
        mm = int(masked[i])
        rows = slice(i * max_m, i * max_m + mm)
        if mm:
            ref32 = orc.fp8_gemm_blockwise(a8[rows], b8[i], a_s[rows], bs[i], 128, 128, layout, out_dtype=None)
            noise = torch.full_like(ref32, float(ref32.abs().max()) * 1e-5)
            check_gemm(out2[i, :mm], ref32, noise, f"masked expert {i} ({mm} rows)")
            assert torch.equal(out[i, :mm], out2[i, :mm])
        assert bool((out2[i, mm:] == marker).all()), f"expert {i}: rows beyond masked_m were written"
