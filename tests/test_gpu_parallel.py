"""GPU (one device): the sharded operators of kernel_set_b200.parallel on the
CUDA library, against the oracle-backed run of the same functions."""
import pytest
import torch

import ks_oracle as orc
from kernel_set_b200 import parallel as par
from test_parallel_cpu import OracleOps, make_linear, make_moe

pytestmark = pytest.mark.gpu


def test_column_shards_on_device(ks, cuda):
    x, w8, ws = make_linear(64, 640, 384, 1)
    ref = par.column_parallel_linear(x, w8, ws, OracleOps())
    parts = []
    for r in range(4):
        w8_s, ws_s, _ = par.shard_weight_columns(w8, ws, r, 4, "nk")
        parts.append(par.column_parallel_linear(x.to(cuda), w8_s.to(cuda), ws_s.to(cuda)).cpu())
    torch.cuda.synchronize()
    assert orc.rel_frobenius(torch.cat(parts, 1).float(), ref.float()) < 1e-3


def test_k_shards_on_device(ks, cuda):
    x, w8, ws = make_linear(32, 256, 1024, 2)
    a8, a_s = orc.quantize_fp8_group(x, 128)
    full32 = orc.fp8_gemm_blockwise(a8, w8, a_s, ws, layout="nk", out_dtype=None)
    total = torch.zeros_like(full32)
    for r in range(2):
        lo, hi = par.block_range(1024, r, 2)
        _, _, b_sh, bs_sh, _ = par.shard_k(a8, a_s, w8, ws, r, 2, "nk")
        q, s = ks.dispatch.per_token_group_quant(x[:, lo:hi].contiguous().to(cuda))
        total += ks.dispatch.fp8_gemm_blockwise(q, b_sh.to(cuda), s, bs_sh.to(cuda), b_layout="nk",
                                                out_dtype=torch.float32).cpu()
    assert orc.rel_frobenius(total, full32) < 1e-5


def test_moe_layer_on_device(ks, cuda):
    x, ids, w, w1, s1, w2, s2 = make_moe(48, 256, 128, 8, 2, 3)
    ref = par.expert_parallel_moe(x, ids, w, w1, s1, w2, s2, 8, OracleOps())
    got = par.expert_parallel_moe(x.to(cuda), ids, w.to(cuda), w1.to(cuda), s1.to(cuda), w2.to(cuda), s2.to(cuda), 8)
    torch.cuda.synchronize()
    ks.runtime.stream_synchronize(0)
    assert orc.rel_frobenius(got.cpu().float(), ref.float()) < 4e-3
