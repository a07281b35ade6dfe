"""GPU: import of GPTQ / AWQ int4 checkpoints (bit-exact against the oracle, which the golden
vectors pin to the provider's packers), and the imported layer through the W4A16 GEMM against
the dense statement of the checkpoint's own arithmetic."""
import pytest
import torch

import ks_oracle as orc
from _util import accumulation_noise, check_gemm, gen, golden

pytestmark = pytest.mark.gpu


def test_golden_checkpoint_imports(ks, cuda):
    g = golden("int4_checkpoint.npz")
    t = {k: torch.from_numpy(v) for k, v in g.items() if getattr(v, "ndim", 0) > 0}
    k, n, gs = int(g["k"]), int(g["n"]), int(g["group_size"])
    want = {"bytes": orc.pack_int4_bytes(t["codes"]), "words": orc.pack_int4_words(t["codes"])}
    for src, name in ((ks.Int4Source.GPTQ, "gptq_qweight"), (ks.Int4Source.AWQ, "awq_qweight")):
        for packing, key in ((ks.Int4Packing.BYTES, "bytes"), (ks.Int4Packing.WORDS, "words")):
            out = torch.empty_like(want[key], device=cuda)
            ks.int4.import_weight(out, t[name].to(cuda), k, n, src, packing)
            assert torch.equal(out.cpu(), want[key]), (name, key)
    for src, name, off, ref in ((ks.Int4Source.GPTQ, "gptq_qzeros_v1", 1, "zeros_gptq"),
                                (ks.Int4Source.GPTQ, "gptq_qzeros_v2", 0, "zeros_awq"),
                                (ks.Int4Source.AWQ, "awq_qzeros", 0, "zeros_awq")):
        for dt in (torch.float32, torch.float16, torch.bfloat16):
            z = torch.empty(k // gs, n, dtype=dt, device=cuda)
            ks.int4.import_zeros(z, t[name].to(cuda), k // gs, n, src, off)
            assert torch.equal(z.cpu().float(), t[ref].float()), (name, dt)
    # activation order through the reference's own entry point
    perm = orc.act_order_perm(t["g_idx"])
    out = torch.empty(k // 2, n, dtype=torch.uint8, device=cuda)
    ks.quant.repack_int4(out, t["gptq_qweight_act_order"].to(cuda), perm.to(cuda), k, n)
    assert torch.equal(out.cpu(), orc.repack_int4(t["gptq_qweight_act_order"], perm))
    assert torch.equal(orc.unpack_int4_bytes(out.cpu()), t["codes"][t["act_order_rows"][perm.long()]])


@pytest.mark.parametrize("k,n", [(4096, 4096), (1024, 11008), (8, 8)])
@pytest.mark.parametrize("source", ["gptq", "awq"])
@pytest.mark.parametrize("with_perm", [False, True])
def test_import_weight_matches_oracle(ks, cuda, k, n, source, with_perm):
    g = gen(k + n)
    codes = torch.randint(0, 16, (k, n), generator=g, dtype=torch.int32)
    qw = orc.gptq_checkpoint(codes, torch.ones(1, n, dtype=torch.int32))[0] if source == "gptq" \
        else orc.awq_checkpoint(codes, torch.zeros(1, n, dtype=torch.int32))[0]
    perm = torch.randperm(k, generator=g).to(torch.int32) if with_perm else None
    src = ks.Int4Source.GPTQ if source == "gptq" else ks.Int4Source.AWQ
    for packing, key, shape, dt in ((ks.Int4Packing.BYTES, "bytes", (k // 2, n), torch.uint8),
                                    (ks.Int4Packing.WORDS, "words", (k // 8, n), torch.int32)):
        out = torch.empty(shape, dtype=dt, device=cuda)
        ks.int4.import_weight(out, qw.to(cuda), k, n, src, packing, perm=perm.to(cuda) if with_perm else None)
        assert torch.equal(out.cpu(), orc.import_int4_weight(qw, source, key, perm))


def test_gather_columns(ks, cuda):
    for rows, cols, dt in ((7, 4096, torch.bfloat16), (1, 24, torch.float32), (33, 1000, torch.float16)):
        g = gen(rows + cols)
        x = torch.randn(rows, cols, generator=g).to(dt)
        perm = torch.randperm(cols, generator=g).to(torch.int32)
        out = torch.empty(rows, cols, dtype=dt, device=cuda)
        ks.int4.gather_columns(out, x.to(cuda), perm.to(cuda), rows, cols)
        assert torch.equal(out.cpu(), x[:, perm.long()])


def _dense_statement(codes, zeros, scales, g_of_row):
    """What the checkpoint means: W[k, n] = (code - zero[g(k)]) * scale[g(k)], rounded to the
    scales' dtype as the W4A16 statement of the reference does."""
    return ((codes.float() - zeros.float()[g_of_row]) * scales.float()[g_of_row]).to(scales.dtype)


@pytest.mark.parametrize("fmt,act_order,m,k,n,gs,dtype", [
    ("gptq", False, 8, 4096, 4096, 128, torch.float16),
    ("gptq", True, 8, 4096, 4096, 128, torch.float16),
    ("gptq", True, 200, 1024, 2048, 128, torch.bfloat16),
    ("awq", False, 8, 4096, 4096, 128, torch.float16),
    ("awq", False, 33, 2048, 11008, 128, torch.bfloat16),
])
def test_imported_layer_equals_dense_statement(ks, cuda, fmt, act_order, m, k, n, gs, dtype):
    g = gen(m + k + n)
    groups = k // gs
    codes = torch.randint(0, 16, (k, n), generator=g, dtype=torch.int32)
    scales = (torch.randn(groups, n, generator=g).mul(0.02).abs() + 1e-3).to(dtype)
    x = torch.randn(m, k, generator=g).to(dtype)
    g_idx = torch.arange(k, dtype=torch.int32) // gs
    if fmt == "gptq":
        zeros = torch.randint(1, 17, (groups, n), generator=g, dtype=torch.int32)
        if act_order:
            g_idx = g_idx[torch.randperm(k, generator=g)].contiguous()
        qw, qz = orc.gptq_checkpoint(codes, zeros, zero_offset=1)
        layer = ks.int4.from_gptq(qw.to(cuda), qz.to(cuda), scales.to(cuda), g_idx.to(cuda), zero_offset=1)
        assert (layer.perm is not None) == act_order
    else:
        zeros = torch.randint(0, 16, (groups, n), generator=g, dtype=torch.int32)
        qw, qz = orc.awq_checkpoint(codes, zeros)
        layer = ks.int4.from_awq(qw.to(cuda), qz.to(cuda), scales.to(cuda))
    out = layer(x.to(cuda))
    torch.cuda.synchronize()
    ks.runtime.stream_synchronize(0)
    w = _dense_statement(codes, zeros, scales, g_idx.long()).float()
    ref32 = x.float() @ w
    check_gemm(out.cpu(), ref32, accumulation_noise(x.float().abs(), w.abs(), k), f"{fmt} layer {m}x{n}x{k}")
    # the imported tensors themselves, bit for bit
    perm = orc.act_order_perm(g_idx) if act_order else None
    assert torch.equal(layer.b_packed.cpu(), orc.import_int4_weight(qw, fmt, "bytes", perm))
    assert torch.equal(layer.zeros.cpu().float(), zeros.float())


def test_import_matches_provider_dequantizer(ks, cuda):
    """Cross-check against the AWQ dequantizer of the provider the reference routes int4 work to,
    when that library is importable: its dense weight equals ours bit for bit."""
    vops = pytest.importorskip("vllm._custom_ops")
    k, n, gs = 1024, 512, 128
    g = gen(9)
    codes = torch.randint(0, 16, (k, n), generator=g, dtype=torch.int32)
    zeros = torch.randint(0, 16, (k // gs, n), generator=g, dtype=torch.int32)
    scales = (torch.rand(k // gs, n, generator=g) * 0.02 + 1e-3).to(torch.float16)
    qw, qz = orc.awq_checkpoint(codes, zeros)
    try:
        theirs = vops.awq_dequantize(qw.to(cuda), scales.to(cuda), qz.to(cuda), 0, 0, 0)
    except Exception as exc:   # the provider has no build of the op for this device
        pytest.skip(f"provider op unavailable: {exc}")
    words = torch.empty(k // 8, n, dtype=torch.int32, device=cuda)
    ks.int4.import_weight(words, qw.to(cuda), k, n, ks.Int4Source.AWQ, ks.Int4Packing.WORDS)
    z = torch.empty(k // gs, n, dtype=torch.float16, device=cuda)
    ks.int4.import_zeros(z, qz.to(cuda), k // gs, n, ks.Int4Source.AWQ, 0)
    ours = torch.empty(k, n, dtype=torch.float16, device=cuda)
    ks.quant.dequantize_int4(ours, words, scales.to(cuda), z, k, n, gs)
    torch.cuda.synchronize()
    assert torch.equal(ours, theirs)
