"""Generates tests/golden/*.npz by running the REFERENCE project's own Python
code on the CPU. Run once in a container that holds a checkout of the
reference (environment variable ``KS_REFERENCE_ROOT``); the tests only read
the frozen vectors.

How the reference is made to run without a GPU:
  * its binding is imported against this repository's library (missing
    symbols are tolerated by the binding's loader); no kernel is executed;
  * torch factory calls with ``device="cuda"`` are redirected to the CPU and
    ``torch.cuda.synchronize`` becomes a no-op for the duration of the script;
  * ``benchmarks/bench.py::_make_fp8_blockwise_inputs`` is called as is: its
    outputs (fp8 codes, scales, dequantized operands) are reference data;
  * for the ops whose torch statement is written inline in a bench function
    (w4a16, int4 dequant, grouped GEMM, the MoE gate / permute / unpermute
    steps, SwiGLU), that function is executed with the
    oracle standing in for the library call. The function then compares the
    stand-in's output with its own inline torch reference and reports
    ``rel_err``; the script insists on exactly 0.0, which proves the oracle
    equals the reference statement bit for bit on those inputs, and freezes
    inputs and outputs.
"""
from __future__ import annotations

import importlib.util
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
REF = os.environ.get("KS_REFERENCE_ROOT")
if not REF:
    raise SystemExit("set KS_REFERENCE_ROOT to a checkout of the reference project")
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "oracle"))
import ks_oracle as orc  # noqa: E402


def _cpu_factories():
    names = ["randn", "randint", "rand", "empty", "zeros", "ones", "full", "arange", "tensor", "empty_like"]
    for name in names:
        orig = getattr(torch, name)

        def wrapped(*a, __orig=orig, **k):
            if str(k.get("device", "")).startswith("cuda"):
                k["device"] = "cpu"
            return __orig(*a, **k)

        setattr(torch, name, wrapped)
    torch.cuda.synchronize = lambda *a, **k: None


def _load_reference_bench():
    os.environ["KERNEL_SET_LIB"] = os.path.join(ROOT, "kernel_set_b200", "lib", "libkernel_set.so")
    sys.path.insert(0, os.path.join(REF, "bindings", "python"))
    spec = importlib.util.spec_from_file_location("ref_bench", os.path.join(REF, "benchmarks", "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    sys.modules["ref_bench"] = mod
    spec.loader.exec_module(mod)
    assert mod._HAVE_KS, mod._KS_IMPORT_ERROR
    fake = types.SimpleNamespace(median_us=1.0, min_us=1.0, p20_us=1.0, p80_us=1.0, method="none", iters=1)
    mod.time_op = lambda fn: fake
    return mod


def u8(t: torch.Tensor) -> np.ndarray:
    return t.view(torch.uint8).numpy().copy()


def bits16(t: torch.Tensor) -> np.ndarray:
    return t.view(torch.int16).numpy().copy()


def main():
    _cpu_factories()
    rb = _load_reference_bench()
    ks = rb.ks
    ctx = rb.Ctx(dt=torch.bfloat16, dtype_name="bf16", gpu=rb.GpuInfo(), warmup=0, iters=1, device="cpu")
    ctx16 = rb.Ctx(dt=torch.float16, dtype_name="fp16", gpu=rb.GpuInfo(), warmup=0, iters=1, device="cpu")

    # ---- FP8 blockwise: reference input preparation and dequantized operands ----
    for tag, (m, n, k) in {"a": (40, 200, 300), "b": (128, 256, 256)}.items():
        torch.manual_seed(11)
        a8, b8, a_s, b_s, a_deq, b_deq = rb._make_fp8_blockwise_inputs(m, n, k, 128, 128)
        torch.manual_seed(11)  # the function's first two draws, in its order
        a_f = torch.randn(m, k, dtype=torch.float32) * 0.1
        b_f = torch.randn(k, n, dtype=torch.float32) * 0.1
        ref = a_deq @ b_deq  # bench.py:1502 before the output rounding
        # oracle == reference on the same inputs, bit for bit
        q, s = orc.quantize_fp8_group(a_f, 128)
        assert torch.equal(s, a_s) and torch.equal(q.view(torch.uint8), a8.view(torch.uint8))
        qb, sb = orc.quantize_weight_blocks(b_f, 128, 128)
        assert torch.equal(sb, b_s) and torch.equal(qb.view(torch.uint8), b8.view(torch.uint8))
        assert torch.equal(orc.dequantize_a(a8, a_s), a_deq) and torch.equal(orc.dequantize_b(b8, b_s), b_deq)
        assert torch.equal(orc.fp8_gemm_blockwise(a8, b8, a_s, b_s, out_dtype=None), ref)
        np.savez_compressed(os.path.join(HERE, f"fp8_blockwise_{tag}.npz"), a_f=a_f.numpy(), b_f=b_f.numpy(),
                            a8=u8(a8), b8=u8(b8), a_scale=a_s.numpy(), b_scale=b_s.numpy(), ref=ref.numpy())
        print("fp8_blockwise", tag, (m, n, k), "oracle == reference")

    # ---- ops whose reference statement is inline: oracle stands in for the kernel ----
    record = {}

    def fake_w4a16(out, a, b_packed, scales, zeros, m, n, k, group_size, **kw):
        out.copy_(orc.w4a16(a, b_packed, scales, zeros, group_size))
        record["w4a16"] = dict(a=bits16(a), b_packed=b_packed.numpy().copy(), scales=bits16(scales),
                               zeros=bits16(zeros), out=bits16(out), group_size=np.int64(group_size),
                               dtype=np.bytes_(str(a.dtype)))
        return out

    def fake_dequant(out, qweight, scales, zeros, k, n, group_size, **kw):
        out.copy_(orc.dequantize_int4(qweight, scales, zeros, group_size, out.dtype))
        record["dequant"] = dict(qweight=qweight.numpy().copy(), scales=bits16(scales), zeros=bits16(zeros),
                                 out=bits16(out), group_size=np.int64(group_size),
                                 repacked=orc.repack_int4(qweight).numpy().copy())
        return out

    def fake_grouped(c, a, b, offsets, E, total_rows, n, k, **kw):
        c.copy_(orc.grouped_gemm(a, b, offsets.tolist()))
        record["grouped"] = dict(a=bits16(a), b=bits16(b), offsets=offsets.numpy().copy(), out=bits16(c))
        return c

    ks.gemm.gemm_w4a16 = fake_w4a16
    ks.quant.dequantize_int4 = fake_dequant
    ks.moe.grouped_gemm = fake_grouped

    for tag, c, (m, n, k, g) in (("bf16", ctx, (16, 192, 256, 128)), ("f16", ctx16, (5, 72, 128, 32))):
        torch.manual_seed(3)
        r = rb._bench_w4a16(c, m, n, k, g)
        assert r.rel_err == 0.0, (tag, r.rel_err, r.status)
        np.savez_compressed(os.path.join(HERE, f"w4a16_{tag}.npz"), **record["w4a16"])
        print("w4a16", tag, "reference bench rel_err", r.rel_err)

    torch.manual_seed(5)
    r = rb._bench_dequantize_int4(ctx, 256, 96, 64)
    assert r.rel_err == 0.0, (r.rel_err, r.status)
    np.savez_compressed(os.path.join(HERE, "int4_dequant_bf16.npz"), **record["dequant"])
    print("dequantize_int4 reference bench rel_err", r.rel_err)

    torch.manual_seed(7)
    r = rb._bench_moe_grouped_gemm(ctx, 24, 96, 80, 4, 2)
    assert r.rel_err == 0.0, (r.rel_err, r.status)
    np.savez_compressed(os.path.join(HERE, "grouped_gemm_bf16.npz"), **record["grouped"])
    print("moe_grouped_gemm reference bench rel_err", r.rel_err)

    # ---- MoE steps around the grouped GEMM, and SwiGLU ----
    def fake_gate(weights, indices, logits, num_tokens, E, k, renormalize=True, **kw):
        w, i = orc.moe_route(logits, k)
        weights.copy_(w)
        indices.copy_(i.to(torch.int32))
        record["gate"] = dict(logits=bits16(logits), weights=weights.numpy().copy(), indices=indices.numpy().copy())
        return weights, indices

    def fake_permutation(sorted_ids, offsets, indices, tokens, E, k, **kw):
        order, off = orc.sort_by_expert(indices.to(torch.int64), E)
        sorted_ids.copy_(order.to(torch.int32))
        offsets.copy_(off)
        record["perm"] = dict(indices=indices.numpy().copy(), sorted_ids=sorted_ids.numpy().copy(),
                              offsets=offsets.numpy().copy())
        return sorted_ids, offsets

    def fake_permute(permuted, x, sorted_ids, tokens, k, hidden, **kw):
        permuted.copy_(orc.moe_permute(x, sorted_ids, k))
        record["permute"] = dict(x=bits16(x), sorted_ids=sorted_ids.numpy().copy(), top_k=np.int64(k),
                                 out=bits16(permuted))
        return permuted

    def fake_unpermute(out, permuted, sorted_ids, weights, tokens, k, hidden, **kw):
        out.copy_(orc.moe_unpermute(permuted, sorted_ids, weights, tokens, k))
        record["unpermute"] = dict(permuted=bits16(permuted), sorted_ids=sorted_ids.numpy().copy(),
                                   weights=weights.numpy().copy(), top_k=np.int64(k), out=bits16(out))
        return out

    def fake_swiglu(out, gate, up, **kw):
        out.copy_(orc.swiglu(gate, up))
        record["swiglu"] = dict(gate=bits16(gate), up=bits16(up), out=bits16(out))
        return out

    ks.moe.gate_softmax_topk = fake_gate
    ks.moe.compute_permutation = fake_permutation
    ks.moe.permute = fake_permute
    ks.moe.unpermute = fake_unpermute
    ks.activation.swiglu = fake_swiglu

    torch.manual_seed(9)
    r = rb._bench_moe_gate(ctx, 48, 0, 0, 16, 4)
    assert r.rel_err == 0.0, (r.rel_err, r.status)
    print("moe_gate reference bench rel_err", r.rel_err)
    torch.manual_seed(10)
    r = rb._bench_moe_permute(ctx, 40, 96, 8, 2)
    assert r.rel_err == 0.0, (r.rel_err, r.status)
    print("moe_permute reference bench rel_err", r.rel_err)
    torch.manual_seed(11)
    r = rb._bench_moe_unpermute(ctx, 40, 96, 8, 2)
    assert r.rel_err == 0.0, (r.rel_err, r.status)
    print("moe_unpermute reference bench rel_err", r.rel_err)
    torch.manual_seed(12)
    r = rb._bench_swiglu(ctx, 24, 160)
    assert r.rel_err == 0.0, (r.rel_err, r.status)
    print("swiglu reference bench rel_err", r.rel_err)
    flat = {f"{op}.{k}": v for op in ("gate", "perm", "permute", "unpermute", "swiglu") for k, v in record[op].items()}
    np.savez_compressed(os.path.join(HERE, "moe_steps_bf16.npz"), **flat)

    abi_symbols()


def abi_symbols():
    """Every function the reference's headers declare, as `<header> <symbol>` lines."""
    import glob
    import re
    rows = []
    for h in sorted(glob.glob(os.path.join(REF, "include", "kernel_set", "*.h"))):
        text = re.sub(r"/\*.*?\*/", "", open(h).read(), flags=re.S)
        rows += [(os.path.basename(h), n) for n in re.findall(r"KS_API[^;(]*?\b(ks_[a-z0-9_]+)\s*\(", text)]
    with open(os.path.join(HERE, "reference_abi_symbols.txt"), "w") as f:
        f.write("# Every function the reference project's headers declare (include/kernel_set/*.h), one per line:\n"
                "# <header> <symbol>. Written by tests/golden/make_golden.py (abi_symbols).\n")
        f.writelines(f"{h} {n}\n" for h, n in rows)
    print("reference ABI:", len(rows), "functions")


if __name__ == "__main__":
    main()
