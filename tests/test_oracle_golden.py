"""CPU: the oracle replayed against the vectors frozen from the reference's own
Python code (tests/golden/make_golden.py), plus the oracle's internal
consistency (its float64 bound, its two statements of the FP8 algebra, the
int4 pack/unpack round trips)."""
import torch

import ks_oracle as orc
from _util import from_bits16, from_u8, golden


def test_fp8_blockwise_inputs_and_gemm_match_reference():
    for tag in ("a", "b"):
        g = golden(f"fp8_blockwise_{tag}.npz")
        a_f, b_f = torch.from_numpy(g["a_f"]), torch.from_numpy(g["b_f"])
        a8, a_s = orc.quantize_fp8_group(a_f, 128)
        b8, b_s = orc.quantize_weight_blocks(b_f, 128, 128)
        assert torch.equal(a8.view(torch.uint8), torch.from_numpy(g["a8"]))
        assert torch.equal(a_s, torch.from_numpy(g["a_scale"]))
        assert torch.equal(b8.view(torch.uint8), torch.from_numpy(g["b8"]))
        assert torch.equal(b_s, torch.from_numpy(g["b_scale"]))
        ref = torch.from_numpy(g["ref"])
        assert torch.equal(orc.fp8_gemm_blockwise(a8, b8, a_s, b_s, out_dtype=None), ref)
        # the [N,K] statement is the same product
        out_nk = orc.fp8_gemm_blockwise(a8, b8.t().contiguous(), a_s, b_s.t().contiguous(), layout="nk",
                                        out_dtype=None)
        assert torch.equal(out_nk, ref)
        # kernel algebra (two-level) and torch statement agree to fp32 noise
        two = orc.fp8_gemm_blockwise_two_level(a8, b8, a_s, b_s)
        assert orc.rel_frobenius(two, ref) < 1e-6
        ref64 = orc.fp8_gemm_blockwise(a8, b8, a_s, b_s, out_dtype=None, acc=torch.float64)
        assert orc.rel_frobenius(ref, ref64) < 1e-6


def test_w4a16_matches_reference():
    for tag, dt in (("bf16", torch.bfloat16), ("f16", torch.float16)):
        g = golden(f"w4a16_{tag}.npz")
        a = from_bits16(g["a"], dt)
        out = orc.w4a16(a, torch.from_numpy(g["b_packed"]), from_bits16(g["scales"], dt),
                        from_bits16(g["zeros"], dt), int(g["group_size"]))
        assert torch.equal(out.view(torch.int16), torch.from_numpy(g["out"]))


def test_int4_dequant_and_repack_match_reference():
    g = golden("int4_dequant_bf16.npz")
    qw = torch.from_numpy(g["qweight"])
    sc, zp = from_bits16(g["scales"], torch.bfloat16), from_bits16(g["zeros"], torch.bfloat16)
    out = orc.dequantize_int4(qw, sc, zp, int(g["group_size"]), torch.bfloat16)
    assert torch.equal(out.view(torch.int16), torch.from_numpy(g["out"]))
    assert torch.equal(orc.repack_int4(qw), torch.from_numpy(g["repacked"]))


def test_grouped_gemm_matches_reference():
    g = golden("grouped_gemm_bf16.npz")
    a, b = from_bits16(g["a"], torch.bfloat16), from_bits16(g["b"], torch.bfloat16)
    out = orc.grouped_gemm(a, b, g["offsets"].tolist())
    assert torch.equal(out.view(torch.int16), torch.from_numpy(g["out"]))


def test_moe_steps_match_reference():
    g = golden("moe_steps_bf16.npz")
    bf = torch.bfloat16
    logits = from_bits16(g["gate.logits"], bf)
    w, i = orc.moe_route(logits, g["gate.indices"].shape[1])
    assert torch.equal(w, torch.from_numpy(g["gate.weights"]))
    assert torch.equal(i.to(torch.int32), torch.from_numpy(g["gate.indices"]))
    ids = torch.from_numpy(g["perm.indices"])
    order, offs = orc.sort_by_expert(ids.to(torch.int64), g["perm.offsets"].shape[0] - 1)
    assert torch.equal(order.to(torch.int32), torch.from_numpy(g["perm.sorted_ids"]))
    assert torch.equal(offs, torch.from_numpy(g["perm.offsets"]))
    x = from_bits16(g["permute.x"], bf)
    out = orc.moe_permute(x, torch.from_numpy(g["permute.sorted_ids"]), int(g["permute.top_k"]))
    assert torch.equal(out.view(torch.int16), torch.from_numpy(g["permute.out"]))
    y = from_bits16(g["unpermute.permuted"], bf)
    k = int(g["unpermute.top_k"])
    out = orc.moe_unpermute(y, torch.from_numpy(g["unpermute.sorted_ids"]), torch.from_numpy(g["unpermute.weights"]),
                            y.shape[0] // k, k)
    assert torch.equal(out.view(torch.int16), torch.from_numpy(g["unpermute.out"]))
    gate, up = from_bits16(g["swiglu.gate"], bf), from_bits16(g["swiglu.up"], bf)
    assert torch.equal(orc.swiglu(gate, up).view(torch.int16), torch.from_numpy(g["swiglu.out"]))
    assert torch.equal(orc.swiglu_packed(torch.cat([gate, up], 1)).view(torch.int16), torch.from_numpy(g["swiglu.out"]))


def test_int4_round_trips():
    gen = torch.Generator().manual_seed(1)
    codes = torch.randint(0, 16, (64, 24), generator=gen).to(torch.int32)
    words = orc.pack_int4_words(codes)
    assert torch.equal(orc.unpack_int4_words(words), codes)
    by = orc.pack_int4_bytes(codes)
    assert torch.equal(orc.unpack_int4_bytes(by), codes)
    assert torch.equal(orc.repack_int4(words), by)
    # byte i of a word is output row 4*word_row + i (what the CUDA repack relies on)
    as_bytes = words.view(torch.uint8).view(8, 24, 4).permute(0, 2, 1).reshape(32, 24)
    assert torch.equal(as_bytes, by)


def test_quantizer_edge_cases():
    x = torch.zeros(3, 200)
    x[1, 5] = 3.0e38
    x[2, 130] = -1e-30
    q, s = orc.quantize_fp8_group(x, 128)
    assert s.shape == (3, 2) and float(s[0, 0]) == 1e-12 or abs(float(s[0, 0]) - 1e-12) < 1e-18
    assert not torch.isnan(q.float()).any()
    assert float(q.float()[1, 5]) == 448.0
    # round trip bound: |x - q*s| <= half an e4m3 step at the group maximum
    g = torch.Generator().manual_seed(2)
    x = torch.randn(16, 512, generator=g).to(torch.bfloat16)
    q, s = orc.quantize_fp8_group(x, 128)
    deq = q.float() * s.repeat_interleave(128, 1)
    assert ((deq - x.float()).abs() <= 0.0625 * x.float().abs().clamp_min(1e-3) + 2.0 ** -10 * s.repeat_interleave(128, 1) * 448).all()


def test_e4m3_cast_saturation_domain():
    # Inside the quantizer |x/scale| never exceeds 448*(1+2^-23), where the
    # non-saturating torch cast and a saturating hardware cast agree.
    v = torch.tensor([447.9, 448.0, 448.00003, 463.9])
    assert torch.equal(v.to(torch.float8_e4m3fn).float(), torch.full((4,), 448.0))


def test_int4_checkpoint_formats_match_provider_packers():
    """The oracle's statement of the GPTQ and AWQ file layouts against vectors packed by the
    provider's own packers (tests/golden/make_int4_checkpoint_golden.py)."""
    g = golden("int4_checkpoint.npz")
    t = {k: torch.from_numpy(v) for k, v in g.items() if getattr(v, "ndim", 0) > 0}
    codes, gs = t["codes"], int(g["group_size"])
    qw, qz1 = orc.gptq_checkpoint(codes, t["zeros_gptq"], zero_offset=1)
    assert torch.equal(qw, t["gptq_qweight"]) and torch.equal(qz1, t["gptq_qzeros_v1"])
    assert torch.equal(orc.gptq_checkpoint(codes, t["zeros_awq"], zero_offset=0)[1], t["gptq_qzeros_v2"])
    aw, az = orc.awq_checkpoint(codes, t["zeros_awq"])
    assert torch.equal(aw, t["awq_qweight"]) and torch.equal(az, t["awq_qzeros"])
    # import: both formats give the same codes and zero-points back, in both packings
    want_bytes, want_words = orc.pack_int4_bytes(codes), orc.pack_int4_words(codes)
    for src, q in (("gptq", t["gptq_qweight"]), ("awq", t["awq_qweight"])):
        assert torch.equal(orc.import_int4_weight(q, src, "bytes"), want_bytes)
        assert torch.equal(orc.import_int4_weight(q, src, "words"), want_words)
    assert torch.equal(orc.import_int4_zeros(t["gptq_qzeros_v1"], "gptq", 1, torch.int32), t["zeros_gptq"])
    assert torch.equal(orc.import_int4_zeros(t["gptq_qzeros_v2"], "gptq", 0, torch.int32), t["zeros_awq"])
    assert torch.equal(orc.import_int4_zeros(t["awq_qzeros"], "awq", 0, torch.int32), t["zeros_awq"])
    # activation order: sorting the stored rows by group gives a layer whose group of row k' is k' // gs,
    # and whose rows are those of the unpermuted layer in the order rows[perm]
    perm = orc.act_order_perm(t["g_idx"])
    assert torch.equal(t["g_idx"][perm.long()].long(), torch.arange(codes.shape[0]) // gs)
    got = orc.unpack_int4_bytes(orc.repack_int4(t["gptq_qweight_act_order"], perm))
    assert torch.equal(got, codes[t["act_order_rows"][perm.long()]])
    assert torch.equal(orc.repack_int4(t["gptq_qweight"]), want_bytes)
