"""GPU: the quantizer fused into its producers and the column-major scale layout.

RMSNorm follows the reference's torch statement (benchmarks/bench.py:877-879) up to the
reciprocal square root and the order of the sum of squares: a last-place difference there can
flip the rounding of the intermediate `T(x * inv_rms)`, which the second rounding after the
weight can widen to two units in the last place of the output, rarely; the fused forms
must equal the unfused library calls run one after the other bit for bit; the GEMM fed with
column-major scales must equal the GEMM fed with row-major ones bit for bit."""
import pytest
import torch

import ks_oracle as orc
from _util import gen, quant_group_device, block_quant_nk_device

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rows,cols,dtype", [
    (4096, 7168, torch.bfloat16),     # the activation of the headline GEMM
    (33, 1024, torch.float16),
    (5, 8192, torch.bfloat16),        # the widest row the register kernel takes
    (7, 200, torch.float32),          # element-wise kernel
    (3, 16384, torch.bfloat16),       # too wide for registers: element-wise kernel
])
def test_rms_norm(ks, cuda, rows, cols, dtype):
    g = gen(rows + cols)
    x = torch.randn(rows, cols, generator=g).to(dtype)
    w = (torch.rand(cols, generator=g) + 0.5).to(dtype)
    out = torch.empty(rows, cols, dtype=dtype, device=cuda)
    ks.norm.rms_norm(out, x.to(cuda), w.to(cuda), eps=1e-6)
    torch.cuda.synchronize()
    ref = orc.rms_norm(x, w, 1e-6).float()
    got = out.cpu().float()
    tol = {torch.float32: 3e-6, torch.float16: 2.1e-3, torch.bfloat16: 1.6e-2}[dtype]   # two units in the last place
    assert float(((got - ref).abs() / (ref.abs() + 1e-3)).max()) < tol
    assert orc.rel_err_max(got, ref) < tol
    if dtype != torch.float32:
        assert (got != ref).float().mean().item() < 0.02, "more than rare last-place differences"


@pytest.mark.parametrize("rows,cols,dtype", [(4096, 7168, torch.bfloat16), (37, 1024, torch.float16),
                                             (2, 8192, torch.bfloat16)])
def test_rms_norm_quant_equals_norm_then_quantize(ks, cuda, rows, cols, dtype):
    g = gen(rows * 3 + cols)
    x = torch.randn(rows, cols, generator=g).to(dtype).to(cuda)
    w = (torch.rand(cols, generator=g) + 0.5).to(dtype).to(cuda)
    q = torch.empty(rows, cols, dtype=torch.float8_e4m3fn, device=cuda)
    s = torch.empty(rows, cols // 128, dtype=torch.float32, device=cuda)
    ks.norm.rms_norm_quant_fp8(q, s, x, w, eps=1e-6)
    y = torch.empty(rows, cols, dtype=dtype, device=cuda)
    ks.norm.rms_norm(y, x, w, eps=1e-6)
    q2, s2 = ks.dispatch.per_token_group_quant(y)
    torch.cuda.synchronize()
    assert torch.equal(q.view(torch.uint8), q2.view(torch.uint8)) and torch.equal(s, s2)
    # and against the oracle's statement of the two steps: the quantizer is exact, so codes
    # differ only where the normalised value itself differs in the last place
    q_ref, s_ref = orc.quantize_fp8_group(orc.rms_norm(x.cpu(), w.cpu(), 1e-6), 128)
    assert (q.cpu().view(torch.uint8) != q_ref.view(torch.uint8)).float().mean().item() < 5e-3
    assert torch.allclose(s.cpu(), s_ref, rtol=1e-2)


@pytest.mark.parametrize("rows,cols,ld,dtype", [(4096, 7168, 4096, torch.bfloat16), (130, 256, 132, torch.float16),
                                                (5, 128, 8, torch.float32),
                                                (1361, 7168, 1364, torch.float16)])
def test_quantizer_column_major_scales(ks, cuda, rows, cols, ld, dtype):
    x = torch.randn(rows, cols, generator=gen(rows + cols + ld)).to(dtype).to(cuda)
    q = torch.empty(rows, cols, dtype=torch.float8_e4m3fn, device=cuda)
    st = torch.full((cols // 128, ld), -1.0, dtype=torch.float32, device=cuda)
    ks.quant.quantize_fp8_group_colscale(q, st, x, rows, cols)
    q2, s2 = ks.dispatch.per_token_group_quant(x)
    torch.cuda.synchronize()
    assert torch.equal(q.view(torch.uint8), q2.view(torch.uint8))
    assert torch.equal(st[:, :rows].t().contiguous(), s2)
    assert bool((st[:, rows:] == -1.0).all()), "padding of the scale rows was written"
    q_ref, s_ref = orc.quantize_fp8_group(x.cpu(), 128)
    assert torch.equal(q.cpu().view(torch.uint8), q_ref.view(torch.uint8)) and torch.equal(s2.cpu(), s_ref)


@pytest.mark.parametrize("m,n,k,layout", [(4096, 7168, 7168, "nk"), (300, 400, 528, "kn"), (2500, 2000, 4096, "nk")])
def test_gemm_with_column_major_scales_equals_row_major(ks, cuda, m, n, k, layout):
    g = torch.Generator(device=cuda).manual_seed(m + n + k)
    a = torch.randn(m, k, generator=g, device=cuda).to(torch.bfloat16)
    if k % 128 == 0:
        b8, b_s = block_quant_nk_device(torch.randn(-(-n // 128) * 128, k, generator=g, device=cuda) * 0.02)
        b8, b_s = b8[:n].contiguous(), b_s
    else:
        w = torch.randn(k, n, generator=gen(3)) * 0.02
        q_kn, s_kn = orc.quantize_weight_blocks(w, 128, 128)
        b8, b_s = q_kn.t().contiguous().to(cuda), s_kn.t().contiguous().to(cuda)
    if layout == "kn":
        b8, b_s = b8.t().contiguous(), b_s.t().contiguous()
    a8, a_s = ks.dispatch.per_token_group_quant(a)
    nkb = -(-k // 128)
    ld = (m + 3) // 4 * 4
    st = torch.zeros(nkb, ld, dtype=torch.float32, device=cuda)
    st[:, :m] = a_s.t()
    out_row = ks.dispatch.fp8_gemm_blockwise(a8, b8, a_s, b_s, b_layout=layout)
    out_col = torch.empty(m, n, dtype=torch.bfloat16, device=cuda)
    ks.gemm.gemm_fp8_blockwise_colscale(out_col, a8, b8, st, b_s, m, n, k, b_layout=layout)
    torch.cuda.synchronize()
    ks.runtime.stream_synchronize(0)
    assert torch.equal(out_row, out_col)
