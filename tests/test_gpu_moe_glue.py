"""GPU: the mixture-of-experts steps around the grouped GEMMs (gate, permutation,
gather / weighted scatter, SwiGLU, and the forms fused with the 1 x 128 quantizer)
through the C ABI against the oracle's restatement of the reference's torch checks
(benchmarks/bench.py:957-958, 1555-1557, 2546-2548, 2570-2579).

Bars: indices, permutations, gathered rows and every fp8 code / scale of the fused
forms bit-exact; routing weights within 2e-6 relative; sums and activations within one
rounding of the output type of the fp32 value."""
import pytest
import torch

import ks_oracle as orc
from _util import gen

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("tokens,experts,top_k,dtype,renorm", [
    (4096, 256, 8, torch.float32, True),      # the MoE configuration of the benchmark
    (4096, 256, 8, torch.bfloat16, True),
    (33, 8, 2, torch.float16, False),
    (5, 1000, 32, torch.float32, True),       # the limits: 1000 experts, top-32
    (1, 4, 4, torch.float32, True),           # every expert chosen
])
def test_gate_softmax_topk(ks, cuda, tokens, experts, top_k, dtype, renorm):
    logits = torch.randn(tokens, experts, generator=gen(tokens + experts)).to(dtype)
    w = torch.empty(tokens, top_k, dtype=torch.float32, device=cuda)
    idx = torch.empty(tokens, top_k, dtype=torch.int32, device=cuda)
    ks.moe.gate_softmax_topk(w, idx, logits.to(cuda), tokens, experts, top_k, renormalize=renorm)
    torch.cuda.synchronize()
    probs = torch.softmax(logits.float(), dim=-1)
    ref_w, ref_i = torch.topk(probs, top_k, dim=-1)
    if renorm:
        ref_w = ref_w / ref_w.sum(-1, keepdim=True)
    w, idx = w.cpu(), idx.cpu().to(torch.int64)
    assert torch.allclose(w, ref_w, rtol=2e-6, atol=1e-9)
    # the same experts in the same order, except between experts of equal probability (16-bit
    # logits repeat values; which of two equal ones is taken at the cut is not specified)
    assert bool((idx >= 0).all()) and bool((idx < experts).all())
    assert all(len(set(row)) == top_k for row in idx.tolist()), "an expert was chosen twice"
    differs = idx != ref_i
    assert torch.equal(probs.gather(1, idx)[differs], probs.gather(1, ref_i)[differs])
    if dtype == torch.float32:
        assert not bool(differs.any())
    assert bool((w[:, :-1] >= w[:, 1:]).all()), "weights are not in descending order"


def test_gate_ties_go_to_the_lowest_expert(ks, cuda):
    logits = torch.zeros(3, 16)
    logits[1, 5] = 1.0
    logits[2, 9:12] = 2.0
    w = torch.empty(3, 4, dtype=torch.float32, device=cuda)
    idx = torch.empty(3, 4, dtype=torch.int32, device=cuda)
    ks.moe.gate_softmax_topk(w, idx, logits.to(cuda), 3, 16, 4, renormalize=True)
    assert idx.cpu().tolist() == [[0, 1, 2, 3], [5, 0, 1, 2], [9, 10, 11, 0]]
    assert torch.allclose(w.cpu().sum(1), torch.ones(3))


def _route(tokens, experts, top_k, seed):
    _, ids = orc.moe_route(torch.randn(tokens, experts, generator=gen(seed)), top_k)
    return ids.to(torch.int32)


@pytest.mark.parametrize("tokens,experts,top_k", [
    (4096, 256, 8),      # 32768 pairs: 1024 per warp
    (3, 4, 2),
    (1000, 7, 3),        # pair count not a multiple of 32, experts not a multiple of anything
    (257, 1000, 5),
])
def test_compute_permutation_is_the_stable_sort(ks, cuda, tokens, experts, top_k):
    ids = _route(tokens, experts, top_k, 3)
    sorted_ids = torch.full((tokens * top_k,), -7, dtype=torch.int32, device=cuda)
    offsets = torch.full((experts + 1,), -7, dtype=torch.int32, device=cuda)
    ks.moe.compute_permutation(sorted_ids, offsets, ids.to(cuda), tokens, experts, top_k)
    torch.cuda.synchronize()
    order, ref_off = orc.sort_by_expert(ids.to(torch.int64), experts)
    assert torch.equal(offsets.cpu(), ref_off)
    assert torch.equal(sorted_ids.cpu().to(torch.int64), order)


def test_compute_permutation_drops_ids_out_of_range(ks, cuda):
    ids = torch.tensor([[0, 3], [9, 1], [-1, 3], [2, 2]], dtype=torch.int32)   # 9 and -1 are not experts (E = 4)
    sorted_ids = torch.empty(8, dtype=torch.int32, device=cuda)
    offsets = torch.empty(5, dtype=torch.int32, device=cuda)
    ks.moe.compute_permutation(sorted_ids, offsets, ids.to(cuda), 4, 4, 2)
    assert offsets.cpu().tolist() == [0, 1, 2, 4, 6]
    assert sorted_ids.cpu().tolist() == [0, 3, 6, 7, 1, 5, -1, -1]


@pytest.mark.parametrize("tokens,hidden,experts,top_k,dtype", [
    (4096, 7168, 256, 8, torch.bfloat16),
    (100, 200, 8, 2, torch.float32),
    (77, 129, 8, 3, torch.float16),          # rows that are not 16-byte multiples: element-wise path
    (64, 256, 16, 4, torch.float8_e4m3fn),
])
def test_permute_gathers_rows(ks, cuda, tokens, hidden, experts, top_k, dtype):
    ids = _route(tokens, experts, top_k, 11)
    order, _ = orc.sort_by_expert(ids.to(torch.int64), experts)
    x = torch.randn(tokens, hidden, generator=gen(5)).to(dtype)
    out = torch.empty(tokens * top_k, hidden, dtype=dtype, device=cuda)
    ks.moe.permute(out, x.to(cuda), order.to(torch.int32).to(cuda), tokens, top_k, hidden)
    torch.cuda.synchronize()
    ref = orc.moe_permute(x.view(torch.uint8) if dtype == torch.float8_e4m3fn else x, order, top_k)
    got = out.cpu()
    assert torch.equal(got.view(torch.uint8) if dtype == torch.float8_e4m3fn else got, ref)


def test_permute_zero_fills_dropped_rows(ks, cuda):
    x = torch.randn(4, 64, generator=gen(1)).to(torch.bfloat16)
    ids = torch.tensor([3, -1, 0, 99], dtype=torch.int32)
    out = torch.empty(4, 64, dtype=torch.bfloat16, device=cuda)
    ks.moe.permute(out, x.to(cuda), ids.to(cuda), 4, 1, 64)
    got = out.cpu()
    assert torch.equal(got[0], x[3]) and torch.equal(got[2], x[0])
    assert not got[1].any() and not got[3].any()


@pytest.mark.parametrize("tokens,hidden,experts,top_k,dtype", [
    (4096, 7168, 256, 8, torch.bfloat16),
    (50, 384, 8, 2, torch.float16),
    (9, 128, 4, 1, torch.float32),
])
def test_permute_quant_equals_permute_then_quantize(ks, cuda, tokens, hidden, experts, top_k, dtype):
    ids = _route(tokens, experts, top_k, 12)
    order, _ = orc.sort_by_expert(ids.to(torch.int64), experts)
    x = torch.randn(tokens, hidden, generator=gen(6)).to(dtype)
    q = torch.empty(tokens * top_k, hidden, dtype=torch.float8_e4m3fn, device=cuda)
    s = torch.empty(tokens * top_k, hidden // 128, dtype=torch.float32, device=cuda)
    ks.moe.permute_quant_fp8(q, s, x.to(cuda), order.to(torch.int32).to(cuda), tokens, top_k, hidden)
    torch.cuda.synchronize()
    rows = 4096 if tokens * top_k > 4096 else tokens * top_k      # the oracle affords a window of the big case
    q_ref, s_ref = orc.quantize_fp8_group(orc.moe_permute(x, order[:rows], top_k), 128)
    assert torch.equal(q.cpu()[:rows].view(torch.uint8), q_ref.view(torch.uint8))
    assert torch.equal(s.cpu()[:rows], s_ref)
    # and the whole output against the two library calls run one after the other
    p = torch.empty(tokens * top_k, hidden, dtype=dtype, device=cuda)
    ks.moe.permute(p, x.to(cuda), order.to(torch.int32).to(cuda), tokens, top_k, hidden)
    q2, s2 = ks.dispatch.per_token_group_quant(p)
    assert torch.equal(q.view(torch.uint8), q2.view(torch.uint8)) and torch.equal(s, s2)


@pytest.mark.parametrize("tokens,hidden,experts,top_k,dtype", [
    (4096, 7168, 256, 8, torch.bfloat16),
    (40, 264, 8, 2, torch.float16),
    (21, 100, 4, 3, torch.float32),
    (16, 99, 4, 2, torch.bfloat16),          # element-wise path
])
def test_unpermute_weighted_sum(ks, cuda, tokens, hidden, experts, top_k, dtype):
    g = gen(13)
    w, ids = orc.moe_route(torch.randn(tokens, experts, generator=g), top_k)
    order, _ = orc.sort_by_expert(ids, experts)
    y = torch.randn(tokens * top_k, hidden, generator=g).to(dtype)
    out = torch.empty(tokens, hidden, dtype=dtype, device=cuda)
    sid = order.to(torch.int32).to(cuda)
    ks.moe.unpermute(out, y.to(cuda), sid, w.to(cuda), tokens, top_k, hidden)
    out2 = torch.empty_like(out)
    ks.moe.unpermute(out2, y.to(cuda), sid, w.to(cuda), tokens, top_k, hidden)   # workspace reused
    torch.cuda.synchronize()
    ref32 = orc.moe_unpermute(y, order, w, tokens, top_k, out_dtype=None)
    got = out.cpu().float()
    tol = {torch.float32: 2e-6, torch.float16: 1.2e-3, torch.bfloat16: 9e-3}[dtype]
    assert float(((got - ref32).abs() / (ref32.abs() + 0.05)).max()) < tol
    assert orc.rel_frobenius(got, ref32) < (1e-6 if dtype == torch.float32 else 3e-3)
    assert torch.equal(out, out2)


def test_unpermute_skips_dropped_pairs(ks, cuda):
    y = torch.ones(4, 32, dtype=torch.bfloat16)
    ids = torch.tensor([0, 3, -1, -1], dtype=torch.int32)        # pairs 1 and 2 were dropped
    w = torch.tensor([[0.25, 0.75], [0.5, 0.5]])
    out = torch.empty(2, 32, dtype=torch.bfloat16, device=cuda)
    ks.moe.unpermute(out, y.to(cuda), ids.to(cuda), w.to(cuda), 2, 2, 32)
    assert out.cpu().float()[:, 0].tolist() == [0.25, 0.5]


@pytest.mark.parametrize("rows,inter,dtype", [
    (4096, 2048, torch.bfloat16),     # between the expert GEMMs of the MoE configuration (per 4096 rows)
    (33, 144, torch.float16),
    (7, 50, torch.float32),           # element-wise path
    (1, 14336, torch.bfloat16),       # a decode row
])
def test_swiglu(ks, cuda, rows, inter, dtype):
    g = gen(rows + inter)
    x = (torch.randn(rows, 2 * inter, generator=g) * 2).to(dtype)
    out = torch.empty(rows, inter, dtype=dtype, device=cuda)
    ks.activation.swiglu_packed(out, x.to(cuda))
    gate, up = x[:, :inter].contiguous(), x[:, inter:].contiguous()
    out2 = torch.empty(rows, inter, dtype=dtype, device=cuda)
    ks.activation.swiglu(out2, gate.to(cuda), up.to(cuda))
    torch.cuda.synchronize()
    assert torch.equal(out, out2)
    ref32 = orc.swiglu_packed(x, out_dtype=None)
    got = out.cpu().float()
    tol = {torch.float32: 2e-6, torch.float16: 1.2e-3, torch.bfloat16: 9e-3}[dtype]
    assert float(((got - ref32).abs() / (ref32.abs() + 1e-3)).max()) < tol
    assert orc.rel_err_max(got, ref32) < tol


@pytest.mark.parametrize("rows,inter,dtype", [(4096, 2048, torch.bfloat16), (37, 256, torch.float16)])
def test_swiglu_quant_equals_swiglu_then_quantize(ks, cuda, rows, inter, dtype):
    x = (torch.randn(rows, 2 * inter, generator=gen(rows)) * 2).to(dtype).to(cuda)
    q = torch.empty(rows, inter, dtype=torch.float8_e4m3fn, device=cuda)
    s = torch.empty(rows, inter // 128, dtype=torch.float32, device=cuda)
    ks.activation.swiglu_packed_quant_fp8(q, s, x)
    act = torch.empty(rows, inter, dtype=dtype, device=cuda)
    ks.activation.swiglu_packed(act, x)
    q2, s2 = ks.dispatch.per_token_group_quant(act)
    torch.cuda.synchronize()
    assert torch.equal(q.view(torch.uint8), q2.view(torch.uint8)) and torch.equal(s, s2)
    # against the oracle: the quantizer is exact, so the codes differ only where the
    # activation itself fell on the other side of a rounding boundary
    q_ref, s_ref = orc.quantize_fp8_group(orc.swiglu_packed(x.cpu()), 128)
    mismatch = (q.cpu().view(torch.uint8) != q_ref.view(torch.uint8)).float().mean().item()
    assert mismatch < 2e-3
    assert torch.allclose(s.cpu(), s_ref, rtol=1e-2)


def test_peer_dispatch_and_combine_on_one_device(ks, cuda):
    """The three steps of the peer-memory dispatch / combine with both "ranks" on one GPU (the
    destination pointers are local tensors): every row must land, bit for bit, where the plan
    says, and come back to the position of the source's sorted order."""
    world, experts, per, tokens, k, hidden = 2, 6, 3, 40, 2, 256
    g = gen(31)
    pairs = tokens * k
    cap = pairs * world
    xs, sorted_ids, offsets, q_loc, s_loc = [], [], [], [], []
    for r in range(world):
        x = torch.randn(tokens, hidden, generator=g).to(torch.bfloat16).to(cuda)
        ids = torch.stack([torch.randperm(experts, generator=g)[:k] for _ in range(tokens)]).to(torch.int32).to(cuda)
        sid = torch.empty(pairs, dtype=torch.int32, device=cuda)
        off = torch.empty(experts + 1, dtype=torch.int32, device=cuda)
        ks.moe.compute_permutation(sid, off, ids, tokens, experts, k)
        q = torch.empty(pairs, hidden, dtype=torch.float8_e4m3fn, device=cuda)
        s = torch.empty(pairs, hidden // 128, dtype=torch.float32, device=cuda)
        ks.moe.permute_quant_fp8(q, s, x, sid, tokens, k, hidden)
        xs.append(x); sorted_ids.append(sid); offsets.append(off); q_loc.append(q); s_loc.append(s)
    counts = torch.stack([o[1:] - o[:-1] for o in offsets]).contiguous()        # [world, experts]
    recv_q = [torch.full((cap, hidden), 0xAA, dtype=torch.uint8, device=cuda) for _ in range(world)]
    recv_s = [torch.full((cap, hidden // 128), -1.0, device=cuda) for _ in range(world)]
    plans = []
    for r in range(world):
        dst_base = torch.empty(experts, dtype=torch.int32, device=cuda)
        local_off = torch.empty(per + 1, dtype=torch.int32, device=cuda)
        seg_start = torch.empty(per * world + 1, dtype=torch.int32, device=cuda)
        ret_base = torch.empty(per * world, dtype=torch.int32, device=cuda)
        ks.moe.dispatch_plan(dst_base, local_off, seg_start, ret_base, counts, world, r, per)
        plans.append((dst_base, local_off, seg_start, ret_base))
        ks.moe.permute_quant_fp8_scatter(recv_q, recv_s, cap, dst_base, offsets[r], experts, per, xs[r], sorted_ids[r],
                                         tokens, k, hidden)
    torch.cuda.synchronize()
    c = counts.cpu()
    offs_h = [o.cpu() for o in offsets]
    for d in range(world):
        local_off = plans[d][1].cpu()
        row = 0
        for el in range(per):
            e = d * per + el
            assert int(local_off[el]) == row
            for s in range(world):
                n = int(c[s, e])
                lo = int(offs_h[s][e])
                assert torch.equal(recv_q[d][row:row + n], q_loc[s][lo:lo + n].view(torch.uint8)), (d, el, s)
                assert torch.equal(recv_s[d][row:row + n], s_loc[s][lo:lo + n]), (d, el, s)
                row += n
        assert int(local_off[per]) == row
        assert bool((recv_q[d][row:] == 0xAA).all()), "rows beyond the received ones were written"
    # the way back
    back = [torch.zeros(pairs, hidden, dtype=torch.bfloat16, device=cuda) for _ in range(world)]
    ys = [torch.randn(cap, hidden, generator=g).to(torch.bfloat16).to(cuda) for _ in range(world)]
    for d in range(world):
        ks.moe.scatter_rows(back, pairs, ys[d], cap, plans[d][2], plans[d][3], per * world, hidden)
    torch.cuda.synchronize()
    for d in range(world):
        row = 0
        for el in range(per):
            e = d * per + el
            for s in range(world):
                n = int(c[s, e])
                lo = int(offs_h[s][e])
                assert torch.equal(back[s][lo:lo + n], ys[d][row:row + n]), (d, el, s)
                row += n
