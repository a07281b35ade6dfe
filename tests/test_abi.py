"""CPU: the shared library loads, exports every symbol the headers declare
(and nothing else with default visibility), answers the introspection calls,
and rejects bad arguments with the reference's status codes before touching
the GPU. No kernel runs here."""
import ctypes
import glob
import os
import re
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    names = []
    for h in sorted(glob.glob(os.path.join(ROOT, "include", "kernel_set", "*.h"))):
        text = open(h).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names += re.findall(r"KS_API[^;(]*?\b(ks_[a-z0-9_]+)\s*\(", text)
    return sorted(set(names))


def test_headers_compile_as_c_and_cpp(tmp_path):
    src = tmp_path / "t.c"
    src.write_text('#include "kernel_set.h"\nint main(void){return (int)KS_DTYPE_I4 - 10;}\n')
    inc = os.path.join(ROOT, "include")
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", "-I", inc, "-fsyntax-only", str(src)], check=True)
    subprocess.run(["g++", "-std=c++17", "-Wall", "-Werror", "-I", inc, "-x", "c++", "-fsyntax-only", str(src)],
                   check=True)


def test_every_declared_symbol_is_exported(ks):
    decl = declared_symbols()
    assert len(decl) == 49, decl
    out = subprocess.run(["nm", "-D", "--defined-only", ks.LIB_PATH], capture_output=True, text=True, check=True)
    exported = sorted(l.split()[-1] for l in out.stdout.splitlines() if " T " in l)
    assert [s for s in decl if s not in exported] == []
    assert [s for s in exported if not s.startswith("ks_")] == [], "non-ABI symbols leak from the library"
    assert ks._lib._MISSING == []


def test_every_reference_symbol_resolves(ks):
    """Bindings that resolve all of the reference's 89 functions when they load (cgo, a Rust
    build script) must link: what this library does not implement answers NOT_IMPLEMENTED."""
    rows = [l.split() for l in open(os.path.join(ROOT, "tests", "golden", "reference_abi_symbols.txt"))
            if l.strip() and not l.startswith("#")]
    assert len(rows) == 89
    ours = set(declared_symbols())
    for header, name in rows:
        fn = getattr(ks._lib.lib, name)          # AttributeError = would not link
        if name not in ours:
            fn.restype = ctypes.c_int
            fn.argtypes = []
            assert fn() == ks.Status.NOT_IMPLEMENTED, name
            assert name in ks.runtime.last_error_string()
    implemented = sorted(n for _, n in rows if n in ours)
    assert len(implemented) == 32 and "ks_moe_unpermute" in implemented and "ks_swiglu_packed" in implemented


def test_introspection(ks):
    lib = ks._lib.lib
    assert ks.version().startswith("0.2.1")
    assert ks.backend_name() == "cuda"
    names = ["KS_SUCCESS", "KS_ERROR_INVALID_ARGUMENT", "KS_ERROR_UNSUPPORTED_DTYPE", "KS_ERROR_UNSUPPORTED_SHAPE",
             "KS_ERROR_CUDA", "KS_ERROR_NOT_IMPLEMENTED", "KS_ERROR_OUT_OF_MEMORY", "KS_ERROR_ARCH_UNSUPPORTED",
             "KS_ERROR_INTERNAL"]
    assert [ks.runtime.status_string(i) for i in range(9)] == names
    assert ks.runtime.status_string(99) == "KS_ERROR_UNKNOWN"
    bits = {0: 32, 1: 16, 2: 16, 3: 8, 4: 8, 5: 64, 6: 64, 7: 32, 8: 8, 9: 8, 10: 4, 77: 0}
    assert {d: ks.runtime.dtype_size_bits(d) for d in bits} == bits
    assert [ks.runtime.dtype_name(d) for d in (0, 1, 2, 3, 4, 10, 55)] == \
        ["f32", "f16", "bf16", "f8e4m3", "f8e5m2", "i4", "unknown"]
    assert lib.ks_last_error_string() is not None


P = ctypes.c_void_p
ONE = P(16)  # a non-NULL token; argument checks never dereference it


def f32p(v):
    return ctypes.cast(v, ctypes.POINTER(ctypes.c_float))


def i32p(v):
    return ctypes.cast(v, ctypes.POINTER(ctypes.c_int32))


def test_argument_validation_codes(ks):
    L = ks._lib.lib
    S = ks.Status
    D = ks.DType
    # ks_quantize_fp8_group (reference quant_fp8_group.cu:137-151)
    assert L.ks_quantize_fp8_group(None, f32p(ONE), ONE, 4, 128, 128, D.BF16, D.F8E4M3, None) == S.INVALID_ARGUMENT
    assert "null arg" in ks.runtime.last_error_string()
    assert L.ks_quantize_fp8_group(ONE, f32p(ONE), ONE, 0, 128, 128, D.BF16, D.F8E4M3, None) == S.INVALID_ARGUMENT
    assert L.ks_quantize_fp8_group(ONE, f32p(ONE), ONE, 4, 128, 0, D.BF16, D.F8E4M3, None) == S.INVALID_ARGUMENT
    assert L.ks_quantize_fp8_group(ONE, f32p(ONE), ONE, 4, 128, 128, D.BF16, D.BF16, None) == S.UNSUPPORTED_DTYPE
    assert L.ks_quantize_fp8_group(ONE, f32p(ONE), ONE, 4, 128, 128, D.I8, D.F8E4M3, None) == S.UNSUPPORTED_DTYPE
    # ks_gemm_fp8_blockwise (reference gemm_fp8_blockwise.cu:224-251)
    args = dict(m=8, n=8, k=8, bn=128, bk=128, f8=D.F8E4M3, odt=D.BF16)

    def bw(fn=L.ks_gemm_fp8_blockwise, out=ONE, a=ONE, b=ONE, sa=ONE, sb=ONE, **kw):
        v = {**args, **kw}
        return fn(out, a, b, f32p(sa), f32p(sb), v["m"], v["n"], v["k"], v["bn"], v["bk"], v["f8"], v["odt"], None)

    for fn in (L.ks_gemm_fp8_blockwise, L.ks_gemm_fp8_blockwise_nt):
        assert bw(fn, out=None) == S.INVALID_ARGUMENT
        assert bw(fn, sb=None) == S.INVALID_ARGUMENT
        assert bw(fn, m=0) == S.INVALID_ARGUMENT
        assert bw(fn, bn=0) == S.INVALID_ARGUMENT
        assert bw(fn, m=2 ** 62, k=4) == S.UNSUPPORTED_SHAPE
        assert bw(fn, f8=D.BF16) == S.UNSUPPORTED_DTYPE
        assert bw(fn, odt=D.I8) == S.UNSUPPORTED_DTYPE
    assert L.ks_gemm_fp8_blockwise(ONE, ONE, ONE, f32p(ONE), f32p(ONE), 8, 8, 8, 128, 128, D.F8E4M3, D.I8, None) \
        == S.UNSUPPORTED_DTYPE
    # ks_gemm_w4a16 (reference gemm_w4a16.cu:156-169)
    w = L.ks_gemm_w4a16
    assert w(None, ONE, ONE, ONE, None, None, 4, 8, 8, 8, D.BF16, None) == S.INVALID_ARGUMENT
    assert w(ONE, ONE, ONE, None, None, None, 4, 8, 8, 8, D.BF16, None) == S.INVALID_ARGUMENT
    assert w(ONE, ONE, ONE, ONE, None, None, 4, 8, 7, 7, D.BF16, None) == S.UNSUPPORTED_SHAPE
    assert w(ONE, ONE, ONE, ONE, None, None, 4, 8, 8, 3, D.BF16, None) == S.UNSUPPORTED_SHAPE
    assert w(ONE, ONE, ONE, ONE, None, None, 4, 8, 8, 8, D.F32, None) == S.UNSUPPORTED_DTYPE
    assert w(ONE, ONE, ONE, ONE, None, None, 0, 8, 8, 8, D.BF16, None) == S.INVALID_ARGUMENT
    # ks_dequantize_int4 / ks_repack_int4 (reference dequant_int4.cu:82-96, repack_int4.cu:46-53)
    dq = L.ks_dequantize_int4
    assert dq(ONE, ONE, ONE, None, 8, 8, 8, D.BF16, None) == S.INVALID_ARGUMENT
    assert dq(ONE, ONE, ONE, ONE, 8, 8, 0, D.BF16, None) == S.INVALID_ARGUMENT
    assert dq(ONE, ONE, ONE, ONE, 12, 8, 4, D.BF16, None) == S.UNSUPPORTED_SHAPE
    assert dq(ONE, ONE, ONE, ONE, 16, 8, 3, D.BF16, None) == S.UNSUPPORTED_SHAPE
    assert dq(ONE, ONE, ONE, ONE, 16, 8, 8, D.I32, None) == S.UNSUPPORTED_DTYPE
    rp = L.ks_repack_int4
    assert rp(ONE, None, None, 8, 8, 4, None) == S.INVALID_ARGUMENT
    assert rp(ONE, ONE, None, 8, 8, 8, None) == S.INVALID_ARGUMENT
    assert rp(ONE, ONE, ONE, 12, 8, 4, None) == S.UNSUPPORTED_SHAPE      # activation order: K, N multiples of 8
    iw, iz, gc = L.ks_int4_import_weight, L.ks_int4_import_zeros, L.ks_gather_columns
    assert iw(ONE, None, None, 8, 8, 0, 0, None) == S.INVALID_ARGUMENT
    assert iw(ONE, ONE, None, 8, 8, 2, 0, None) == S.INVALID_ARGUMENT
    assert iw(ONE, ONE, None, 8, 8, 0, 2, None) == S.INVALID_ARGUMENT
    assert iw(ONE, ONE, None, 12, 8, 0, 0, None) == S.UNSUPPORTED_SHAPE
    assert iz(ONE, ONE, 1, 8, 0, 2, D.F16, None) == S.INVALID_ARGUMENT
    assert iz(ONE, ONE, 1, 12, 0, 1, D.F16, None) == S.UNSUPPORTED_SHAPE
    assert iz(ONE, ONE, 1, 8, 0, 1, D.I32, None) == S.UNSUPPORTED_DTYPE
    assert gc(P(32), ONE, None, 1, 8, D.F16, None) == S.INVALID_ARGUMENT
    assert gc(ONE, ONE, ONE, 1, 8, D.F16, None) == S.INVALID_ARGUMENT        # out aliases input
    assert gc(P(32), ONE, ONE, 1, 8, D.I8, None) == S.UNSUPPORTED_DTYPE
    assert gc(P(32), ONE, ONE, 70000, 8, D.F16, None) == S.UNSUPPORTED_SHAPE
    # scattered GEMM output and the sum of K-split parts
    import ctypes
    two = (ctypes.c_void_p * 2)(16, 32)
    sc, sp = L.ks_gemm_fp8_blockwise_scatter, L.ks_sum_parts
    assert sc(None, 2, 128, ONE, ONE, f32p(ONE), f32p(ONE), 256, 128, 128, 1, D.F8E4M3, D.BF16, None) == S.INVALID_ARGUMENT
    assert sc(two, 9, 128, ONE, ONE, f32p(ONE), f32p(ONE), 256, 128, 128, 1, D.F8E4M3, D.BF16, None) == S.INVALID_ARGUMENT
    assert sc(two, 2, 100, ONE, ONE, f32p(ONE), f32p(ONE), 200, 128, 128, 1, D.F8E4M3, D.BF16, None) == S.UNSUPPORTED_SHAPE
    assert sc(two, 2, 128, ONE, ONE, f32p(ONE), f32p(ONE), 384, 128, 128, 1, D.F8E4M3, D.BF16, None) == S.UNSUPPORTED_SHAPE
    assert sp(two, 0, ONE, 2, 8, 8, D.F32, D.BF16, None) == S.INVALID_ARGUMENT
    assert sp(two, 2, ONE, 2, 8, 8, D.I8, D.BF16, None) == S.UNSUPPORTED_DTYPE
    assert sp(two, 2, ONE, 2, 3, 3, D.F32, D.BF16, None) == S.UNSUPPORTED_SHAPE
    # expert-parallel dispatch / combine through peer memory
    dp, pqs, sr = L.ks_moe_dispatch_plan, L.ks_moe_permute_quant_fp8_scatter, L.ks_moe_scatter_rows
    assert dp(i32p(ONE), i32p(ONE), i32p(ONE), i32p(ONE), i32p(None), 2, 0, 4, None) == S.INVALID_ARGUMENT
    assert dp(i32p(ONE), i32p(ONE), i32p(ONE), i32p(ONE), i32p(ONE), 9, 0, 4, None) == S.INVALID_ARGUMENT
    assert dp(i32p(ONE), i32p(ONE), i32p(ONE), i32p(ONE), i32p(ONE), 2, 2, 4, None) == S.INVALID_ARGUMENT
    assert dp(i32p(ONE), i32p(ONE), i32p(ONE), i32p(ONE), i32p(ONE), 8, 0, 200, None) == S.UNSUPPORTED_SHAPE
    assert pqs(two, two, 2, 64, i32p(ONE), i32p(ONE), 8, 4, ONE, i32p(ONE), 4, 2, 100, D.BF16, D.F8E4M3, None) \
        == S.UNSUPPORTED_SHAPE
    assert pqs(two, two, 2, 64, i32p(ONE), i32p(ONE), 8, 2, ONE, i32p(ONE), 4, 2, 128, D.BF16, D.F8E4M3, None) \
        == S.INVALID_ARGUMENT      # 8 experts, 2 per rank, but only 2 ranks
    assert pqs(two, two, 2, 64, i32p(ONE), i32p(ONE), 8, 4, ONE, i32p(ONE), 4, 2, 128, D.I8, D.F8E4M3, None) \
        == S.UNSUPPORTED_DTYPE
    assert sr(two, 2, 8, ONE, 8, i32p(ONE), i32p(ONE), 3, 128, D.BF16, None) == S.INVALID_ARGUMENT   # 3 segments, 2 ranks
    assert sr(two, 2, 8, ONE, 8, i32p(ONE), i32p(ONE), 4, 4, D.BF16, None) == S.UNSUPPORTED_SHAPE
    assert sr(two, 2, 8, ONE, 8, i32p(ONE), i32p(ONE), 4, 128, D.I32, None) == S.UNSUPPORTED_DTYPE
    # ks_moe_grouped_gemm (reference moe_grouped_gemm.cu:140-153)
    gg = L.ks_moe_grouped_gemm
    assert gg(ONE, ONE, ONE, i32p(None), 2, 8, 8, 8, D.BF16, None) == S.INVALID_ARGUMENT
    assert gg(ONE, ONE, ONE, i32p(ONE), 0, 8, 8, 8, D.BF16, None) == S.INVALID_ARGUMENT
    assert gg(ONE, ONE, ONE, i32p(ONE), 2, 0, 8, 8, D.BF16, None) == S.SUCCESS
    assert gg(ONE, ONE, ONE, i32p(ONE), 2, 8, 8, 8, D.I32, None) == S.UNSUPPORTED_DTYPE
    gf = L.ks_moe_grouped_gemm_fp8_blockwise
    assert gf(ONE, ONE, ONE, f32p(ONE), f32p(ONE), i32p(ONE), 2, 0, 8, 8, 128, 128, 1, D.F8E4M3, D.BF16, None) \
        == S.SUCCESS
    assert gf(ONE, ONE, ONE, f32p(ONE), f32p(ONE), i32p(ONE), 2, 8, 8, 8, 128, 128, 5, D.F8E4M3, D.BF16, None) \
        == S.INVALID_ARGUMENT
    # MoE steps (reference moe_gate.cu / moe_permute.cu launchers) and SwiGLU
    assert L.ks_moe_gate_softmax_topk(f32p(ONE), i32p(ONE), None, 4, 8, 2, 1, D.BF16, None) == S.INVALID_ARGUMENT
    assert L.ks_moe_gate_softmax_topk(f32p(ONE), i32p(ONE), ONE, 4, 8, 9, 1, D.BF16, None) == S.INVALID_ARGUMENT
    assert L.ks_moe_gate_softmax_topk(f32p(ONE), i32p(ONE), ONE, 4, 2000, 2, 1, D.BF16, None) == S.UNSUPPORTED_SHAPE
    assert L.ks_moe_gate_softmax_topk(f32p(ONE), i32p(ONE), ONE, 4, 8, 2, 1, D.I8, None) == S.UNSUPPORTED_DTYPE
    assert L.ks_moe_gate_softmax_topk(f32p(ONE), i32p(ONE), ONE, 0, 8, 2, 1, D.BF16, None) == S.SUCCESS
    assert L.ks_moe_compute_permutation(i32p(ONE), i32p(ONE), i32p(None), 4, 8, 2, None) == S.INVALID_ARGUMENT
    assert L.ks_moe_compute_permutation(i32p(ONE), i32p(ONE), i32p(ONE), 2 ** 31, 8, 2, None) == S.UNSUPPORTED_SHAPE
    assert L.ks_moe_permute(ONE, ONE, i32p(ONE), 4, 0, 8, D.BF16, None) == S.INVALID_ARGUMENT
    assert L.ks_moe_permute(ONE, ONE, i32p(ONE), 4, 2, 8, D.I32, None) == S.UNSUPPORTED_DTYPE
    assert L.ks_moe_permute(ONE, ONE, i32p(ONE), 0, 2, 8, D.BF16, None) == S.SUCCESS
    assert L.ks_moe_permute_quant_fp8(ONE, f32p(ONE), ONE, i32p(ONE), 4, 2, 100, D.BF16, D.F8E4M3, None) \
        == S.UNSUPPORTED_SHAPE
    assert L.ks_moe_unpermute(ONE, ONE, i32p(ONE), f32p(None), 4, 2, 8, D.BF16, None) == S.INVALID_ARGUMENT
    assert L.ks_moe_unpermute(ONE, ONE, i32p(ONE), f32p(ONE), 4, 2, 8, D.F8E4M3, None) == S.UNSUPPORTED_DTYPE
    assert L.ks_swiglu_packed(ONE, None, 4, 8, D.BF16, None) == S.INVALID_ARGUMENT
    assert L.ks_swiglu(ONE, ONE, ONE, 4, 0, D.BF16, None) == S.INVALID_ARGUMENT
    assert L.ks_swiglu(ONE, ONE, ONE, 4, 8, D.I8, None) == S.UNSUPPORTED_DTYPE
    assert L.ks_swiglu_packed_quant_fp8(ONE, f32p(ONE), ONE, 4, 100, D.BF16, D.F8E4M3, None) == S.UNSUPPORTED_SHAPE
    # runtime
    assert L.ks_device_count(None) == S.INVALID_ARGUMENT
    assert L.ks_memcpy(None, ONE, 4, 0, None) == S.INVALID_ARGUMENT


def test_python_marshalling_rejects_host_tensors(ks):
    import torch
    with pytest.raises(ValueError, match="CUDA tensor"):
        ks.dispatch.per_token_group_quant(torch.zeros(2, 128, dtype=torch.bfloat16))
    with pytest.raises(ValueError, match="b_layout"):
        ks.gemm.gemm_fp8_blockwise(1, 1, 1, 1, 1, 1, 1, 1, fp8_dtype=3, out_dtype=2, b_layout="xx")
    with pytest.raises(KeyError):
        ks.dispatch.which("attention_prefill")
    assert ks.dispatch.which("fp8_gemm_blockwise") == "kernel-set"
    assert ks.dispatch.providers("w4a16") == ["kernel-set"]
    assert set(ks.dispatch.available()) == {"fp8_gemm_blockwise", "per_token_group_quant", "w4a16", "moe"}
    assert ks.dispatch.chain("moe", gpu=100)[0]["selectable"] is True
    assert ks.dispatch.Backend("w4a16").name == "kernel-set"
    assert ks.dispatch.per_token_group_quant_fp8 is ks.dispatch.per_token_group_quant
    e = ks.KernelSetError(3, "KS_ERROR_UNSUPPORTED_SHAPE", "msg", "ks_x")
    assert e.status == 3 and "ks_x failed" in str(e)
