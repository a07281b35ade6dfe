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


def _nccl_worker(rank, world, port, q):
    import os
    import sys
    here = os.path.dirname(os.path.abspath(__file__))
    for p in (os.path.dirname(here), os.path.join(os.path.dirname(here), "oracle"), here):
        if p not in sys.path:
            sys.path.insert(0, p)
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from test_parallel_cpu import dense_moe_reference
        # row-parallel linear: K split over the ranks, bf16 partials all-reduced over NCCL
        x, w8, ws = make_linear(64, 512, 2048, 2)
        lo, hi = par.block_range(2048, rank, world)
        a8, a_s = orc.quantize_fp8_group(x, 128)
        _, _, b_sh, bs_sh, _ = par.shard_k(a8, a_s, w8, ws, rank, world, "nk")
        out = par.row_parallel_linear(x[:, lo:hi].contiguous().to(dev), b_sh.to(dev), bs_sh.to(dev))
        torch.cuda.synchronize()
        full32 = orc.fp8_gemm_blockwise(a8, w8, a_s, ws, layout="nk", out_dtype=None)
        frob_row = orc.rel_frobenius(out.float().cpu(), full32)
        # the same layer with the all-reduce fused into the GEMM over peer memory (fp32 slots,
        # summed in rank order): bf16 rounding of the fp32 sum, identical on both ranks and
        # from call to call
        xf, w8f, wsf = make_linear(256, 512, 2048, 3)
        a8f, a_sf = orc.quantize_fp8_group(xf, 128)
        _, _, bf_sh, bsf_sh, _ = par.shard_k(a8f, a_sf, w8f, wsf, rank, world, "nk")
        fused = par.FusedRowParallel(256, 512, device=dev)
        xs = xf[:, lo:hi].contiguous().to(dev)
        out_f = fused(xs, bf_sh.to(dev), bsf_sh.to(dev)).clone()
        out_f2 = fused(xs, bf_sh.to(dev), bsf_sh.to(dev)).clone()
        torch.cuda.synchronize()
        fullf = orc.fp8_gemm_blockwise(a8f, w8f, a_sf, wsf, layout="nk", out_dtype=None)
        frob_fused = orc.rel_frobenius(out_f.float().cpu(), fullf.to(torch.bfloat16).float())
        same = bool(torch.equal(out_f, out_f2))
        gathered = [torch.empty_like(out_f) for _ in range(world)]
        dist.all_gather(gathered, out_f)
        same = same and all(bool(torch.equal(g, out_f)) for g in gathered)
        # expert-parallel MoE: tokens and experts both split, fp8 rows through all_to_all
        xm, ids, w, w1, s1, w2, s2 = make_moe(64, 256, 128, 8, 2, 3)
        t = 64 // world
        t_lo, t_hi = rank * t, (rank + 1) * t
        e_lo, e_hi = par.expert_range(8, rank, world)
        got = par.expert_parallel_moe(xm[t_lo:t_hi].to(dev), ids[t_lo:t_hi].to(dev), w[t_lo:t_hi].to(dev),
                                      w1[e_lo:e_hi].to(dev), s1[e_lo:e_hi].to(dev), w2[e_lo:e_hi].to(dev),
                                      s2[e_lo:e_hi].to(dev), 8)
        torch.cuda.synchronize()
        ref = dense_moe_reference(xm, ids, w, w1, s1, w2, s2)[t_lo:t_hi]
        frob_moe = orc.rel_frobenius(got.float().cpu(), ref.float())
        # the same layer with dispatch and combine as peer stores: same kernels on the same rows in
        # the same order, so the same bits; twice, to go through the buffers' reuse
        layer = par.FusedExpertParallel(t, 2, 256, 128, 8, device=dev)
        margs = (xm[t_lo:t_hi].to(dev), ids[t_lo:t_hi].to(dev), w[t_lo:t_hi].to(dev), w1[e_lo:e_hi].to(dev),
                 s1[e_lo:e_hi].to(dev), w2[e_lo:e_hi].to(dev), s2[e_lo:e_hi].to(dev))
        got_f = layer(*margs).clone()
        got_f2 = layer(*margs).clone()
        torch.cuda.synchronize()
        same = same and bool(torch.equal(got_f, got)) and bool(torch.equal(got_f2, got))
        q.put((rank, float(frob_row), float(frob_moe), float(frob_fused), same))
    finally:
        dist.destroy_process_group()


def test_nccl_world2_row_parallel_and_expert_parallel(ks, cuda):
    """Two ranks on two GPUs over NCCL: the all-reduce of the row-parallel linear and the
    all-to-all dispatch / combine of the expert-parallel layer against the oracle on the
    unsplit problem. Needs two devices; a one-GPU machine skips it."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    from test_parallel_cpu import _free_port
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_nccl_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = sorted(q.get(timeout=300) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, frob_row, frob_moe, frob_fused, same in results:
        # two bf16 partials rounded before the sum and once after: a few 1e-3 at most
        assert frob_row < 4e-3, (rank, frob_row)
        assert frob_moe < 4e-3, (rank, frob_moe)
        # fp32 slots: only the order of the fp32 additions differs from the unsplit product, which
        # flips the final bf16 rounding of a few outputs
        assert frob_fused < 1e-4, (rank, frob_fused)
        assert same, "a fused (peer-memory) path differs between calls, between ranks or from the NCCL path"


def test_scattered_gemm_output_equals_plain(ks, cuda):
    """ks_gemm_fp8_blockwise_scatter into four local buffers: row block b of the plain GEMM,
    bit for bit, in bf16 and in fp32."""
    g = torch.Generator(device=cuda).manual_seed(5)
    m, n, k = 1024, 768, 1024
    a = torch.randn(m, k, generator=g, device=cuda).to(torch.bfloat16)
    w = torch.randn(n, k, generator=g, device=cuda) * 0.02
    from _util import block_quant_nk_device
    b8, b_s = block_quant_nk_device(w)
    a8, a_s = ks.dispatch.per_token_group_quant(a)
    for dt in (torch.bfloat16, torch.float32):
        plain = torch.empty(m, n, dtype=dt, device=cuda)
        ks.gemm.gemm_fp8_blockwise(plain, a8, b8, a_s, b_s, m, n, k, b_layout="nk")
        parts = [torch.full((m // 4, n), -7.0, dtype=dt, device=cuda) for _ in range(4)]
        ks.gemm.gemm_fp8_blockwise_scatter(parts, a8, b8, a_s, b_s, m, n, k, m // 4, b_layout="nk")
        torch.cuda.synchronize()
        for b in range(4):
            assert torch.equal(parts[b], plain[b * (m // 4):(b + 1) * (m // 4)]), (dt, b)
    with pytest.raises(ks.KernelSetError):
        ks.gemm.gemm_fp8_blockwise_scatter(parts[:3], a8, b8, a_s, b_s, m, n, k, m // 4, b_layout="nk")


@pytest.mark.parametrize("part_dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_sum_parts(ks, cuda, part_dtype):
    g = torch.Generator(device=cuda).manual_seed(6)
    parts = torch.randn(3, 40, 200, generator=g, device=cuda).to(part_dtype)
    want32 = (parts[0].float() + parts[1].float()) + parts[2].float()
    for out_dtype in (torch.bfloat16, torch.float32):
        dsts = [torch.empty(40, 200, dtype=out_dtype, device=cuda) for _ in range(2)]
        ks.gemm.sum_parts(dsts, parts, 3, 40, 200)
        torch.cuda.synchronize()
        assert torch.equal(dsts[0], want32.to(out_dtype)) and torch.equal(dsts[1], dsts[0])
