"""GPU: the allocation-free W4A16 entry point (``ks_gemm_w4a16_static_scratch``).

Some hosts of this library may not allocate at run time: a serving engine that
gave the whole GPU to its own memory pool, a decode loop that bans allocator
calls once it is live, a sandbox that lets a plugin only launch and copy. For
them the kernel's split-K scratch is a fixed array inside the library instead of
memory from the CUDA allocator. This file checks, through the C ABI, that the
variant returns what ``ks_gemm_w4a16`` returns, on two calls in a row (the
array keeps the first call's contents when the second starts), and that a shape
too large for the array is refused instead of overrunning it.

The file sorts last on purpose: a run that stops at the first failure has then
already run every other test.
"""
import ctypes

import pytest
import torch

import ks_oracle as orc
from _util import accumulation_noise, check_gemm, gen

pytestmark = pytest.mark.gpu


def _inputs(m, k, n, dtype, seed):
    g = gen(seed)
    a = torch.randn(m, k, generator=g).to(dtype)
    codes = torch.randint(0, 16, (k, n), generator=g).to(torch.int32)
    scales = (torch.randn(k // 128, n, generator=g).mul(0.02).abs() + 1e-3).to(dtype)
    zeros = torch.full((k // 128, n), 8.0).to(dtype)
    bias = torch.randn(n, generator=g).to(dtype)
    return a, orc.pack_int4_bytes(codes), scales, zeros, bias


def _call(ks, symbol, c, a, bp, sc, zp, bias, m, n, k, dtype_id):
    fn = getattr(ks._lib.lib, symbol)
    stream = torch.cuda.current_stream(c.device).cuda_stream
    return fn(c.data_ptr(), a.data_ptr(), bp.data_ptr(), sc.data_ptr(), zp.data_ptr(), bias.data_ptr(),
              m, n, k, 128, dtype_id, ctypes.c_void_p(stream))


@pytest.mark.parametrize("m,k,n,dtype", [
    (8, 4096, 512, torch.bfloat16),    # every column tile split over many thread blocks -> scratch in use
    (32, 2048, 1024, torch.float16),
])
def test_static_scratch_matches_allocating_entry_point(ks, cuda, m, k, n, dtype):
    dtype_id = ks.DType.BF16 if dtype == torch.bfloat16 else ks.DType.F16
    first_out = None
    for call in range(2):
        # different data on the second call: stale slots or counters would show
        a, bp, sc, zp, bias = _inputs(m, k, n, dtype, seed=100 + call)
        dev = [t.to(cuda) for t in (a, bp, sc, zp, bias)]
        c_ref = torch.empty(m, n, dtype=dtype, device=cuda)
        c_new = torch.full((m, n), float("nan"), dtype=dtype, device=cuda)
        assert _call(ks, "ks_gemm_w4a16", c_ref, *dev, m, n, k, dtype_id) == 0, ks.runtime.last_error_string()
        assert _call(ks, "ks_gemm_w4a16_static_scratch", c_new, *dev, m, n, k, dtype_id) == 0, \
            ks.runtime.last_error_string()
        torch.cuda.synchronize()
        ks.runtime.stream_synchronize(0)
        # same kernel, same slot-ordered reduction: the two entry points agree to the bit ...
        assert torch.equal(c_new.view(torch.int16), c_ref.view(torch.int16))
        # ... and both meet the acceptance bound against the oracle
        ref32 = orc.w4a16(a, bp, sc, zp, 128, bias, out_dtype=None)
        noise = accumulation_noise(a.float().abs(), orc.w4a16_weight(bp, sc, zp, 128).float().abs(), k)
        check_gemm(c_new.cpu(), ref32, noise, f"static scratch call {call}")
        if first_out is None:
            first_out = c_new.clone()
    assert not torch.equal(first_out, c_new), "the two calls were meant to differ"


def test_static_scratch_refuses_oversized_shapes(ks, cuda):
    # 224 column tiles x 128 token rows need far more than the 16 MiB array
    m, k, n = 128, 4096, 28672
    a = torch.zeros(m, k, dtype=torch.bfloat16, device=cuda)
    bp = torch.zeros(k // 2, n, dtype=torch.uint8, device=cuda)
    sc = torch.ones(k // 128, n, dtype=torch.bfloat16, device=cuda)
    c = torch.empty(m, n, dtype=torch.bfloat16, device=cuda)
    with pytest.raises(ks.KernelSetError) as ei:
        ks.gemm.gemm_w4a16_static_scratch(c, a, bp, sc, None, m, n, k, 128)
    assert ei.value.status == ks.Status.UNSUPPORTED_SHAPE
    assert "scratch" in ei.value.backend_message
    # the allocating entry point takes the same shape
    ks.gemm.gemm_w4a16(c, a, bp, sc, None, m, n, k, 128)
    torch.cuda.synchronize()
