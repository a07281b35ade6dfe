"""CPU: the sharding and exchange logic of kernel_set_b200.parallel, with the
oracle standing in for the per-device kernels. Single-process checks plus
world-size-2 gloo runs (spawned children, 127.0.0.1 rendezvous)."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import ks_oracle as orc
from kernel_set_b200 import parallel as par


class OracleOps:
    def quant(self, x, group_size=128):
        return orc.quantize_fp8_group(x, group_size)

    def fp8_gemm(self, a8, b8, a_scale, b_scale, b_layout="nk", out_dtype=torch.bfloat16):
        return orc.fp8_gemm_blockwise(a8, b8, a_scale, b_scale, layout=b_layout, out_dtype=out_dtype)

    def grouped_fp8_gemm(self, a8, b8, expert_offsets, a_scale, b_scale, n, k, b_layout="nk"):
        return orc.grouped_gemm_fp8_blockwise(a8, b8, a_scale, b_scale, expert_offsets.tolist(), layout=b_layout)

    def permutation(self, topk_ids, num_experts):
        order, offsets = orc.sort_by_expert(topk_ids.to(torch.int64), num_experts)
        return order.to(torch.int32), offsets

    def permute_quant(self, x, sorted_ids, top_k):
        return orc.quantize_fp8_group(orc.moe_permute(x, sorted_ids, top_k), 128)

    def gather_rows(self, x, index):
        if x.dtype in (torch.float8_e4m3fn, torch.float8_e5m2):
            return x.view(torch.uint8)[index.to(torch.int64)].view(x.dtype)
        return x[index.to(torch.int64)]

    def swiglu_quant(self, gate_up):
        return orc.quantize_fp8_group(orc.swiglu_packed(gate_up), 128)

    def unpermute(self, y, sorted_ids, weights, num_tokens, top_k):
        return orc.moe_unpermute(y, sorted_ids, weights, num_tokens, top_k)


def test_block_range_covers_everything_in_whole_blocks():
    for total in (7168, 896, 300, 128, 100):
        for world in (1, 2, 3, 4, 8):
            spans = [par.block_range(total, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            for (a0, a1), (b0, b1) in zip(spans, spans[1:]):
                assert a1 == b0 and a0 <= a1
            for lo, hi in spans:
                assert (lo % 128 == 0 or lo == total) and (hi % 128 == 0 or hi == total)


def make_linear(m, n, k, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16)
    w_nk = torch.randn(n, k, generator=g) * 0.02
    b8_kn, bs_kn = orc.quantize_weight_blocks(w_nk.t())
    return x, b8_kn.t().contiguous(), bs_kn.t().contiguous()


def test_column_parallel_equals_unsharded():
    x, w8, ws = make_linear(24, 640, 384, 1)
    full = par.column_parallel_linear(x, w8, ws, OracleOps())
    for world in (2, 4):
        parts = []
        for r in range(world):
            w8_s, ws_s, (lo, hi) = par.shard_weight_columns(w8, ws, r, world, "nk")
            assert w8_s.shape[0] == hi - lo
            parts.append(par.column_parallel_linear(x, w8_s, ws_s, OracleOps()))
        # CPU matmuls of different widths block their sums differently: equal up to a bf16 rounding flip
        assert orc.rel_frobenius(torch.cat(parts, dim=1).float(), full.float()) < 1e-3


def test_k_shards_sum_to_unsharded():
    x, w8, ws = make_linear(16, 256, 1024, 2)
    a8, a_s = orc.quantize_fp8_group(x, 128)
    full32 = orc.fp8_gemm_blockwise(a8, w8, a_s, ws, layout="nk", out_dtype=None)
    for world in (2, 4):
        total = torch.zeros_like(full32)
        for r in range(world):
            a_sh, as_sh, b_sh, bs_sh, (lo, hi) = par.shard_k(a8, a_s, w8, ws, r, world, "nk")
            # quantizing the K-slice of the activation gives the same codes as slicing the quantized one
            q_sh, s_sh = orc.quantize_fp8_group(x[:, lo:hi].contiguous(), 128)
            assert torch.equal(q_sh.view(torch.uint8), a_sh.view(torch.uint8)) and torch.equal(s_sh, as_sh)
            total += orc.fp8_gemm_blockwise(a_sh, b_sh, as_sh, bs_sh, layout="nk", out_dtype=None)
        assert orc.rel_frobenius(total, full32) < 1e-6


def make_moe(tokens, hidden, inter, experts, topk, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(tokens, hidden, generator=g).to(torch.bfloat16)
    w, ids = orc.moe_route(torch.randn(tokens, experts, generator=g), topk)
    w1, s1, w2, s2 = [], [], [], []
    for _ in range(experts):
        a, b = orc.quantize_weight_blocks((torch.randn(2 * inter, hidden, generator=g) * 0.02).t())
        w1.append(a.t().contiguous()); s1.append(b.t().contiguous())
        a, b = orc.quantize_weight_blocks((torch.randn(hidden, inter, generator=g) * 0.02).t())
        w2.append(a.t().contiguous()); s2.append(b.t().contiguous())
    return x, ids, w, torch.stack(w1), torch.stack(s1), torch.stack(w2), torch.stack(s2)


def dense_moe_reference(x, ids, w, w1, s1, w2, s2):
    """Token by token, expert by expert, no sorting: what the sharded path must equal."""
    out = torch.zeros(x.shape[0], x.shape[1], dtype=torch.float32)
    for t in range(x.shape[0]):
        for slot in range(ids.shape[1]):
            e = int(ids[t, slot])
            xt = x[t:t + 1]
            x8, xs = orc.quantize_fp8_group(xt, 128)
            h = orc.fp8_gemm_blockwise(x8, w1[e], xs, s1[e], layout="nk")
            a = par.swiglu(h)
            a8, a_s = orc.quantize_fp8_group(a, 128)
            y = orc.fp8_gemm_blockwise(a8, w2[e], a_s, s2[e], layout="nk")
            out[t] += float(w[t, slot]) * y[0].float()
    return out.to(torch.bfloat16)


def test_moe_single_rank_equals_dense_reference():
    x, ids, w, w1, s1, w2, s2 = make_moe(12, 256, 128, 8, 2, 3)
    got = par.expert_parallel_moe(x, ids, w, w1, s1, w2, s2, 8, OracleOps())
    ref = dense_moe_reference(x, ids, w, w1, s1, w2, s2)
    assert orc.rel_frobenius(got.float(), ref.float()) < 4e-3


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, q):
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "oracle"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # row-parallel linear: K split, one all-reduce (fp32 here so that the sum is order-exact)
        x, w8, ws = make_linear(16, 256, 1024, 2)
        lo, hi = par.block_range(1024, rank, world)
        a8, a_s = orc.quantize_fp8_group(x, 128)
        _, _, b_sh, bs_sh, _ = par.shard_k(a8, a_s, w8, ws, rank, world, "nk")
        out = par.row_parallel_linear(x[:, lo:hi].contiguous(), b_sh, bs_sh, OracleOps(), reduce_dtype=torch.float32)
        full32 = orc.fp8_gemm_blockwise(a8, w8, a_s, ws, layout="nk", out_dtype=None)
        ok_row = orc.rel_frobenius(out, full32) < 1e-6
        # expert-parallel MoE: tokens and experts both split over the ranks
        xm, ids, w, w1, s1, w2, s2 = make_moe(12, 256, 128, 8, 2, 3)
        t_lo, t_hi = rank * 6, rank * 6 + 6
        e_lo, e_hi = par.expert_range(8, rank, world)
        got = par.expert_parallel_moe(xm[t_lo:t_hi], ids[t_lo:t_hi], w[t_lo:t_hi], w1[e_lo:e_hi], s1[e_lo:e_hi],
                                      w2[e_lo:e_hi], s2[e_lo:e_hi], 8, OracleOps())
        ref = dense_moe_reference(xm, ids, w, w1, s1, w2, s2)[t_lo:t_hi]
        ok_moe = orc.rel_frobenius(got.float(), ref.float()) < 4e-3
        q.put((rank, bool(ok_row), bool(ok_moe)))
    finally:
        dist.destroy_process_group()


def test_gloo_world2_row_parallel_and_expert_parallel():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=240) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(results) == [(0, True, True), (1, True, True)]


def test_received_to_expert_major_matches_a_plain_sort():
    g = torch.Generator().manual_seed(5)
    for world, per in ((1, 4), (2, 3), (4, 5)):
        counts = torch.randint(0, 4, (world, per), generator=g)
        counts[0, 0] = 0
        total = int(counts.sum())
        # label every arriving row with its local expert, in arrival order (source-major)
        labels = torch.cat([torch.full((int(counts[r, e]),), e) for r in range(world) for e in range(per)]) \
            if total else torch.zeros(0, dtype=torch.int64)
        perm, offsets = par.received_to_expert_major(counts, total)
        assert perm.dtype == torch.int32 and offsets.dtype == torch.int32
        expect = torch.sort(labels, stable=True).indices
        assert torch.equal(perm.to(torch.int64), expect)
        assert offsets.tolist() == [0] + torch.cumsum(counts.sum(0), 0).tolist()
