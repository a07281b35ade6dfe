"""GPU: quantizer and int4 helpers, through the C ABI (via the ctypes binding),
bit-exact against the oracle and the frozen reference vectors."""
import pytest
import torch

import ks_oracle as orc
from _util import from_bits16, gen, golden

pytestmark = pytest.mark.gpu


def run_quant(ks, x_cpu, gs, fp8, dev):
    out, scale = ks.dispatch.per_token_group_quant(x_cpu.to(dev), group_size=gs,
                                                   fp8_dtype=ks.DType.F8E5M2 if fp8 == "e5m2" else None)
    torch.cuda.synchronize()
    return out.cpu(), scale.cpu()


@pytest.mark.parametrize("rows,cols,gs,dtype,fp8", [
    (64, 7168, 128, torch.bfloat16, "e4m3"),    # fast kernel, DeepSeek hidden size
    (37, 2048, 128, torch.float16, "e4m3"),
    (8, 512, 128, torch.float32, "e4m3"),
    (16, 1024, 128, torch.bfloat16, "e5m2"),
    (33, 1000, 128, torch.bfloat16, "e4m3"),    # ragged last group -> general kernel
    (17, 384, 64, torch.float16, "e4m3"),       # other group size
    (5, 700, 300, torch.float32, "e5m2"),       # group larger than a warp pass
    (1, 1, 128, torch.bfloat16, "e4m3"),
    (3, 129, 128, torch.bfloat16, "e4m3"),      # odd width: unaligned rows
    (1361, 7168, 128, torch.float16, "e5m2"),   # several generations of blocks, a partly filled last one
])
def test_quantizer_bit_exact(ks, cuda, rows, cols, gs, dtype, fp8):
    x = (torch.randn(rows, cols, generator=gen(rows * 131 + cols)) * 3.0).to(dtype)
    x[0, :min(cols, gs)] = 0  # an all-zero group exercises the 1e-12 floor
    q_ref, s_ref = orc.quantize_fp8_group(x, gs, fp8)
    q, s = run_quant(ks, x, gs, fp8, cuda)
    assert torch.equal(s, s_ref)
    assert torch.equal(q.view(torch.uint8), q_ref.view(torch.uint8))


def test_quantizer_extreme_values(ks, cuda):
    x = torch.zeros(4, 256, dtype=torch.float32)
    x[0, 3] = 3.0e38
    x[0, 4] = -3.0e38
    x[1, 130] = 1e-30
    x[2, :] = torch.linspace(-448, 448, 256)
    x[3, :] = 2.0 ** -20
    q_ref, s_ref = orc.quantize_fp8_group(x, 128)
    q, s = run_quant(ks, x, 128, "e4m3", cuda)
    assert torch.equal(s, s_ref)
    assert torch.equal(q.view(torch.uint8), q_ref.view(torch.uint8))
    assert not torch.isnan(q.float()).any()


def test_quantizer_deepseek_shape_full(ks, cuda):
    """[4096, 7168] bf16 ~N(0,1): the activation of the headline GEMM, every code and scale."""
    x = torch.randn(4096, 7168, generator=gen(0)).to(torch.bfloat16)
    q_ref, s_ref = orc.quantize_fp8_group(x, 128)
    q, s = run_quant(ks, x, 128, "e4m3", cuda)
    assert torch.equal(s, s_ref)
    assert torch.equal(q.view(torch.uint8), q_ref.view(torch.uint8))


def test_quantizer_rounding_boundaries(ks, cuda):
    """Quotients that sit on, just below and just above the midpoints between fp8 codes,
    for thousands of different scales: any error in the last bit of x / scale shows."""
    g = gen(77)
    groups = 4096
    codes = torch.arange(0, 127, dtype=torch.uint8).view(torch.float8_e4m3fn).float()   # 0 .. 448
    mids = (codes[:-1] + codes[1:]) / 2
    amax = torch.exp(torch.rand(groups, generator=g) * 30.0 - 15.0).float()              # 3e-7 .. 3e6
    scale = torch.clamp(amax / 448.0, min=1e-12)
    pick = torch.randint(0, mids.numel(), (groups, 127), generator=g)
    x = scale[:, None] * mids[pick]
    nudge = torch.randint(-1, 2, (groups, 127), generator=g)
    up = torch.nextafter(x, torch.full_like(x, float("inf")))
    down = torch.nextafter(x, torch.full_like(x, -float("inf")))
    x = torch.where(nudge > 0, up, torch.where(nudge < 0, down, x))
    sign = torch.randint(0, 2, (groups, 127), generator=g).float() * 2 - 1
    x = torch.cat([amax[:, None], x * sign], dim=1).reshape(groups // 8, 8 * 128).contiguous()
    q_ref, s_ref = orc.quantize_fp8_group(x, 128)
    q, s = run_quant(ks, x, 128, "e4m3", cuda)
    assert torch.equal(s, s_ref)
    assert torch.equal(q.view(torch.uint8), q_ref.view(torch.uint8))


def test_quantizer_bf16_patterns(ks, cuda):
    """Random bf16 bit patterns (every mantissa, a 12-binade window per group, windows from
    2^-40 to 2^40): exercises the quotient path far from the N(0,1) activations."""
    g = gen(78)
    groups = 8192
    e0 = torch.randint(127 - 40, 127 + 40, (groups, 1), generator=g)
    expo = e0 - torch.randint(0, 12, (groups, 128), generator=g)
    mant = torch.randint(0, 128, (groups, 128), generator=g)
    sign = torch.randint(0, 2, (groups, 128), generator=g)
    bits = (sign << 15) | (expo << 7) | mant
    x = bits.to(torch.int32).to(torch.int16).view(torch.bfloat16).reshape(groups // 16, 16 * 128).contiguous()
    q_ref, s_ref = orc.quantize_fp8_group(x, 128)
    q, s = run_quant(ks, x, 128, "e4m3", cuda)
    assert torch.equal(s, s_ref)
    assert torch.equal(q.view(torch.uint8), q_ref.view(torch.uint8))


@pytest.mark.parametrize("fp8", ["e4m3", "e5m2"])
def test_quantizer_every_bf16_maximum(ks, cuda, fp8):
    """Every non-negative finite bf16 value as a group's maximum (32 640 groups): the scale is
    amax / qmax for each of them, and the codes of a few fractions of it."""
    bits = torch.arange(0, 0x7F80, dtype=torch.int32)
    amax = bits.to(torch.int16).view(torch.bfloat16)
    x = torch.zeros(bits.numel(), 128, dtype=torch.bfloat16)
    x[:, 0] = amax
    frac = torch.tensor([0.5, -0.75, 0.3, -0.11, 0.97, 1.0 / 3], dtype=torch.float32)
    x[:, 1:7] = (amax.float()[:, None] * frac[None, :]).to(torch.bfloat16)
    x = x.reshape(-1, 16 * 128).contiguous()
    q_ref, s_ref = orc.quantize_fp8_group(x, 128, fp8)
    q, s = run_quant(ks, x, 128, fp8, cuda)
    assert torch.equal(s, s_ref)
    assert torch.equal(q.view(torch.uint8), q_ref.view(torch.uint8))


def test_quantizer_golden(ks, cuda):
    for tag in ("a", "b"):
        g = golden(f"fp8_blockwise_{tag}.npz")
        q, s = run_quant(ks, torch.from_numpy(g["a_f"]), 128, "e4m3", cuda)
        assert torch.equal(q.view(torch.uint8), torch.from_numpy(g["a8"]))
        assert torch.equal(s, torch.from_numpy(g["a_scale"]))


@pytest.mark.parametrize("k,n,gs,dtype", [
    (4096, 4096, 128, torch.bfloat16),   # the CPU-runnable configuration's weight
    (256, 96, 64, torch.float16),
    (64, 30, 16, torch.float32),         # N % 4 != 0 -> scalar kernel
    (128, 8, 128, torch.bfloat16),
])
def test_int4_dequant_and_repack_bit_exact(ks, cuda, k, n, gs, dtype):
    g = gen(k + n)
    codes = torch.randint(0, 16, (k, n), generator=g).to(torch.int32)
    qw = orc.pack_int4_words(codes)
    scales = (torch.randn(k // gs, n, generator=g).mul(0.02).abs() + 1e-3).to(dtype)
    zeros = torch.randint(0, 16, (k // gs, n), generator=g).to(dtype)
    out = torch.empty(k, n, dtype=dtype, device=cuda)
    ks.quant.dequantize_int4(out, qw.to(cuda), scales.to(cuda), zeros.to(cuda), k, n, gs)
    packed = torch.empty(k // 2, n, dtype=torch.uint8, device=cuda)
    ks.quant.repack_int4(packed, qw.to(cuda), None, k, n)
    torch.cuda.synchronize()
    ref = orc.dequantize_int4(qw, scales, zeros, gs, dtype)
    assert torch.equal(out.cpu().view(torch.uint8), ref.view(torch.uint8))
    assert torch.equal(packed.cpu(), orc.repack_int4(qw))
    assert torch.equal(orc.unpack_int4_bytes(packed.cpu()), codes)


def test_int4_golden(ks, cuda):
    g = golden("int4_dequant_bf16.npz")
    qw = torch.from_numpy(g["qweight"])
    k, n = qw.shape[0] * 8, qw.shape[1]
    sc, zp = from_bits16(g["scales"], torch.bfloat16), from_bits16(g["zeros"], torch.bfloat16)
    out = torch.empty(k, n, dtype=torch.bfloat16, device=cuda)
    ks.quant.dequantize_int4(out, qw.to(cuda), sc.to(cuda), zp.to(cuda), k, n, int(g["group_size"]))
    packed = torch.empty(k // 2, n, dtype=torch.uint8, device=cuda)
    ks.quant.repack_int4(packed, qw.to(cuda), None, k, n)
    torch.cuda.synchronize()
    assert torch.equal(out.cpu().view(torch.int16), torch.from_numpy(g["out"]))
    assert torch.equal(packed.cpu(), torch.from_numpy(g["repacked"]))


def test_status_codes_on_device(ks, cuda):
    x = torch.zeros(4, 128, dtype=torch.bfloat16, device=cuda)
    with pytest.raises(ks.KernelSetError) as ei:
        ks.quant.quantize_fp8_group(torch.empty(4, 128, dtype=torch.uint8, device=cuda),
                                    torch.empty(4, 1, device=cuda), x, 4, 128, group_size=0)
    assert ei.value.status == ks.Status.INVALID_ARGUMENT and "group_size" in ei.value.backend_message
    with pytest.raises(ks.KernelSetError) as ei:
        # activation order wants K and N in multiples of 8 (the reference refuses it altogether)
        ks.quant.repack_int4(torch.empty(6, 8, dtype=torch.uint8, device=cuda),
                             torch.zeros(2, 8, dtype=torch.int32, device=cuda),
                             torch.zeros(12, dtype=torch.int32, device=cuda), 12, 8)
    assert ei.value.status == ks.Status.UNSUPPORTED_SHAPE
    with pytest.raises(ValueError, match="contiguous"):
        ks.dispatch.per_token_group_quant(torch.zeros(128, 8, dtype=torch.bfloat16, device=cuda).t())
    assert ks.device_count() >= 1
    props = ks.runtime.get_device_properties(0)
    assert props["compute_major"] == 10 and props["multiprocessor_count"] > 0
