"""Sharding of the quantized GEMMs over the GPUs of one node.

The reference project has no multi-GPU code; these helpers implement the three
partitionings its benchmark definition names, one process per GPU over
``torch.distributed``:

* column-parallel (split N): every rank holds whole 128-column blocks of the
  weight and the matching b_scale rows/columns; activations are replicated;
  no collective, outputs stay sharded ``[M, N/g]``.
* row-parallel (split K): every rank holds whole 128-deep K-blocks of both
  operands and scales; partial products are summed with one all-reduce.
* expert-parallel: experts are split contiguously; tokens travel to the rank
  that owns their expert with ``all_to_all_single`` and back after the
  grouped GEMM.

All index arithmetic is pure (usable on CPU tensors, tested under gloo); only
the GEMM calls need a GPU.
"""
from __future__ import annotations

from typing import List, Sequence, Tuple

import torch
import torch.distributed as dist

BLOCK = 128


def block_range(total: int, rank: int, world: int, block: int = BLOCK) -> Tuple[int, int]:
    """Contiguous [lo, hi) of `total` owned by `rank`, in whole blocks; the first
    ``nblocks % world`` ranks get one block more. hi is clipped to `total`."""
    nblocks = -(-total // block)
    base, extra = divmod(nblocks, world)
    lo_b = rank * base + min(rank, extra)
    hi_b = lo_b + base + (1 if rank < extra else 0)
    return min(lo_b * block, total), min(hi_b * block, total)


# ------------------------------ column-parallel ------------------------------
def shard_weight_columns(b8: torch.Tensor, b_scale: torch.Tensor, rank: int, world: int, layout: str = "nk"):
    """Rank's slice of a block-quantized weight split along N.
    layout "nk": b8 [N,K], b_scale [N/128, K/128]; "kn": b8 [K,N], b_scale [K/128, N/128]."""
    n = b8.shape[0] if layout == "nk" else b8.shape[1]
    lo, hi = block_range(n, rank, world)
    slo, shi = lo // BLOCK, -(-hi // BLOCK)
    if layout == "nk":
        return b8[lo:hi].contiguous(), b_scale[slo:shi].contiguous(), (lo, hi)
    return b8[:, lo:hi].contiguous(), b_scale[:, slo:shi].contiguous(), (lo, hi)


# -------------------------------- row-parallel --------------------------------
def shard_k(a8: torch.Tensor, a_scale: torch.Tensor, b8: torch.Tensor, b_scale: torch.Tensor, rank: int,
            world: int, layout: str = "nk"):
    """Rank's K-slice of both operands and their scales (whole 128-deep blocks)."""
    k = a8.shape[1]
    lo, hi = block_range(k, rank, world)
    slo, shi = lo // BLOCK, -(-hi // BLOCK)
    a_sh, as_sh = a8[:, lo:hi].contiguous(), a_scale[:, slo:shi].contiguous()
    if layout == "nk":
        return a_sh, as_sh, b8[:, lo:hi].contiguous(), b_scale[:, slo:shi].contiguous(), (lo, hi)
    return a_sh, as_sh, b8[lo:hi].contiguous(), b_scale[slo:shi].contiguous(), (lo, hi)


def all_reduce_partials(partial: torch.Tensor, group=None) -> torch.Tensor:
    """Sum of the ranks' partial outputs, in place (NCCL over NVLink on GPUs)."""
    dist.all_reduce(partial, op=dist.ReduceOp.SUM, group=group)
    return partial


# ------------------------------- expert-parallel -------------------------------
def expert_range(num_experts: int, rank: int, world: int) -> Tuple[int, int]:
    per = -(-num_experts // world)
    return min(rank * per, num_experts), min((rank + 1) * per, num_experts)


def exchange_counts(per_expert_counts: torch.Tensor, num_experts: int, world: int, group=None) -> torch.Tensor:
    """All ranks' per-expert counts for the experts this rank owns:
    returns [world, experts_per_rank] (row r = what rank r sends here)."""
    per = -(-num_experts // world)
    pad = per * world - num_experts
    c = per_expert_counts.to(torch.int64)
    if pad:
        c = torch.cat([c, c.new_zeros(pad)])
    recv = torch.empty_like(c)
    dist.all_to_all_single(recv, c, group=group)
    return recv.view(world, per)


def all_to_all_rows(rows: torch.Tensor, send_counts: Sequence[int], recv_counts: Sequence[int], group=None):
    """Variable-size exchange of matrix rows (dim 0)."""
    out = rows.new_empty((int(sum(recv_counts)),) + tuple(rows.shape[1:]))
    dist.all_to_all_single(out, rows.contiguous(), output_split_sizes=[int(v) for v in recv_counts],
                           input_split_sizes=[int(v) for v in send_counts], group=group)
    return out


def received_to_expert_major(recv_counts_matrix: torch.Tensor, total: int):
    """Rows arrive grouped by source rank, and inside a source by local expert.
    Returns (perm, offsets) on the matrix's device, computed without a host read:
    ``received[perm]`` is sorted by local expert (source-rank order inside an
    expert), ``offsets`` int32 [E_local+1]. ``total`` is the number of rows."""
    world, per = recv_counts_matrix.shape
    dev = recv_counts_matrix.device
    c = recv_counts_matrix.to(torch.int64)
    flat = c.reshape(-1)                                            # source-major: how the rows lie
    src_start_em = (torch.cumsum(flat, 0) - flat).view(world, per).t().contiguous().reshape(-1)
    c_em = c.t().contiguous().reshape(-1)                           # expert-major: how they should lie
    dst_start_em = torch.cumsum(c_em, 0) - c_em
    block = torch.repeat_interleave(torch.arange(per * world, device=dev), c_em, output_size=int(total))
    perm = src_start_em[block] + (torch.arange(int(total), device=dev) - dst_start_em[block])
    offsets = torch.zeros(per + 1, dtype=torch.int32, device=dev)
    offsets[1:] = torch.cumsum(c.sum(0), 0).to(torch.int32)
    return perm.to(torch.int32), offsets


# ------------------------------------------------------------------------------
# Sharded operators. `ops` supplies the single-device kernels:
#   ops.quant(x, group_size) -> (codes, scales)
#   ops.fp8_gemm(a8, b8, a_scale, b_scale, b_layout, out_dtype) -> out
#   ops.grouped_fp8_gemm(a8, b8, expert_offsets, a_scale, b_scale, n, k, b_layout) -> out
#   ops.permutation(topk_ids int32 [T,k], num_experts) -> (sorted_token_ids, expert_offsets)
#   ops.permute_quant(x, sorted_token_ids, top_k) -> (codes, scales) of the gathered rows
#   ops.gather_rows(x, index int32) -> x[index]
#   ops.swiglu_quant(gate_up) -> (codes, scales) of silu(gate) * up
#   ops.unpermute(y, sorted_token_ids, weights, num_tokens, top_k) -> weighted sum per token
# The default is this library (CUDA tensors, every step a kernel on the current
# stream, no host round trip). Anything with the same methods can stand in,
# which is how the CPU tests drive the sharding logic.
# ------------------------------------------------------------------------------
class LibraryOps:
    """The CUDA library as the per-device backend of the sharded operators."""

    def quant(self, x, group_size=BLOCK):
        from . import dispatch
        return dispatch.per_token_group_quant(x, group_size=group_size)

    def fp8_gemm(self, a8, b8, a_scale, b_scale, b_layout="nk", out_dtype=torch.bfloat16):
        from . import dispatch
        return dispatch.fp8_gemm_blockwise(a8, b8, a_scale, b_scale, b_layout=b_layout, out_dtype=out_dtype)

    def grouped_fp8_gemm(self, a8, b8, expert_offsets, a_scale, b_scale, n, k, b_layout="nk"):
        from . import dispatch
        return dispatch.moe(a8, b8, expert_offsets, n=n, k=k, a_scale=a_scale, b_scale=b_scale, b_layout=b_layout)

    def permutation(self, topk_ids, num_experts):
        from . import moe
        t, k = topk_ids.shape
        sorted_ids = torch.empty(t * k, dtype=torch.int32, device=topk_ids.device)
        offsets = torch.empty(num_experts + 1, dtype=torch.int32, device=topk_ids.device)
        return moe.compute_permutation(sorted_ids, offsets, topk_ids, t, num_experts, k)

    def permute_quant(self, x, sorted_ids, top_k):
        from . import moe
        t, hidden = x.shape
        out = torch.empty(t * top_k, hidden, dtype=torch.float8_e4m3fn, device=x.device)
        scale = torch.empty(t * top_k, hidden // BLOCK, dtype=torch.float32, device=x.device)
        return moe.permute_quant_fp8(out, scale, x, sorted_ids, t, top_k, hidden)

    def gather_rows(self, x, index):
        from . import moe
        out = torch.empty_like(x)
        if x.shape[0]:
            moe.permute(out, x, index, x.shape[0], 1, x.shape[1])
        return out

    def swiglu_quant(self, gate_up):
        from . import activation
        rows, two_inter = gate_up.shape
        out = torch.empty(rows, two_inter // 2, dtype=torch.float8_e4m3fn, device=gate_up.device)
        scale = torch.empty(rows, two_inter // 2 // BLOCK, dtype=torch.float32, device=gate_up.device)
        return activation.swiglu_packed_quant_fp8(out, scale, gate_up, rows, two_inter // 2)

    def unpermute(self, y, sorted_ids, weights, num_tokens, top_k):
        from . import moe
        out = torch.empty(num_tokens, y.shape[1], dtype=y.dtype, device=y.device)
        return moe.unpermute(out, y, sorted_ids, weights, num_tokens, top_k, y.shape[1])


def column_parallel_linear(x: torch.Tensor, w8_shard: torch.Tensor, ws_shard: torch.Tensor, ops=None,
                           b_layout: str = "nk") -> torch.Tensor:
    """x [M,K] (replicated) times this rank's column shard of the weight: quantize
    locally, multiply, keep the output sharded [M, N/g]. No collective."""
    ops = ops or LibraryOps()
    a8, a_s = ops.quant(x, BLOCK)
    return ops.fp8_gemm(a8, w8_shard, a_s, ws_shard, b_layout, torch.bfloat16)


def row_parallel_linear(x_shard: torch.Tensor, w8_kshard: torch.Tensor, ws_kshard: torch.Tensor, ops=None,
                        b_layout: str = "nk", group=None, reduce_dtype=torch.bfloat16) -> torch.Tensor:
    """x_shard [M, K/g] (this rank's K-slice of the activation) times this rank's
    K-slice of the weight, then one all-reduce of the partial outputs. The 1 x 128
    activation groups never straddle ranks because K-slices are whole blocks."""
    ops = ops or LibraryOps()
    a8, a_s = ops.quant(x_shard, BLOCK)
    partial = ops.fp8_gemm(a8, w8_kshard, a_s, ws_kshard, b_layout, reduce_dtype)
    return all_reduce_partials(partial, group)


class FusedRowParallel:
    """Row-parallel linear whose all-reduce runs inside the GEMM and one summing kernel, over
    peer memory, instead of as a collective behind the GEMM.

    Rank ``r`` owns the output rows ``[r * m / g, (r + 1) * m / g)``. Every rank's GEMM writes
    its partial product of row block ``b`` straight into rank ``b``'s memory (TMA stores of
    the finished tiles, ``ks_gemm_fp8_blockwise_scatter``), so the reduce-scatter's traffic
    crosses NVLink while later tiles are still being computed. After a barrier each rank adds
    the ``g`` slots of its rows in rank order in fp32 (``ks_sum_parts``: the same bits on
    every run, and one rounding instead of the ``g`` of a bf16 all-reduce) and writes the
    result into every rank's output buffer, which is the all-gather. A second barrier ends
    the step. Buffers come from ``torch.distributed._symmetric_memory``.

    The returned tensor is owned by this object and is overwritten by the next call.
    """

    def __init__(self, m: int, n: int, group=None, part_dtype=torch.float32, device=None):
        import torch.distributed._symmetric_memory as symm_mem
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        if m % (BLOCK * self.world) != 0:
            raise ValueError("m must be a multiple of 128 * world size")
        self.m, self.n, self.rows = m, n, m // self.world
        device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.parts = symm_mem.empty((self.world, self.rows, n), dtype=part_dtype, device=device)
        self.final = symm_mem.empty((m, n), dtype=torch.bfloat16, device=device)
        self.h_parts = symm_mem.rendezvous(self.parts, self.group)
        self.h_final = symm_mem.rendezvous(self.final, self.group)
        slot = self.rows * n
        # where this rank's partial of row block b goes: slot `rank` of rank b's parts
        self.part_ptrs = [int(self.h_parts.buffer_ptrs[b]) + self.rank * slot * self.parts.element_size()
                          for b in range(self.world)]
        # where this rank's finished rows go in every rank's output
        self.final_ptrs = [int(self.h_final.buffer_ptrs[b]) + self.rank * slot * 2 for b in range(self.world)]

    def __call__(self, x_shard: torch.Tensor, w8_kshard: torch.Tensor, ws_kshard: torch.Tensor, ops=None,
                 gather: bool = True) -> torch.Tensor:
        from . import gemm
        from ._tensor import dtype_to_ks
        ops = ops or LibraryOps()
        a8, a_s = ops.quant(x_shard, BLOCK)
        return self.multiply(a8, a_s, w8_kshard, ws_kshard, gather)

    def multiply(self, a8, a_s, w8_kshard, ws_kshard, gather: bool = True) -> torch.Tensor:
        from . import gemm
        from ._tensor import dtype_to_ks
        k_local = a8.shape[1]
        gemm.gemm_fp8_blockwise_scatter(self.part_ptrs, a8, w8_kshard, a_s, ws_kshard, self.m, self.n, k_local,
                                        self.rows, out_dtype=dtype_to_ks(self.parts.dtype), b_layout="nk")
        self.h_parts.barrier()   # every rank's slot of my rows has landed
        dsts = self.final_ptrs if gather else [self.final_ptrs[self.rank]]
        gemm.sum_parts(dsts, self.parts, self.world, self.rows, self.n, out_dtype=dtype_to_ks(torch.bfloat16))
        self.h_final.barrier()   # every rank's rows have landed in my output; nobody reads parts any more
        return self.final if gather else self.final[self.rank * self.rows:(self.rank + 1) * self.rows]


class FusedExpertParallel:
    """Expert-parallel MoE layer whose dispatch and combine are peer stores of the kernels that
    produce the rows, instead of all-to-all collectives with a regrouping pass on either side.

    Steps on every rank: counting-sort permutation; all-gather of the per-expert counts (small,
    on the device); ``ks_moe_dispatch_plan``; gather + 1 x 128 quantizer writing every row into
    its destination rank's buffer at its final expert-major position
    (``ks_moe_permute_quant_fp8_scatter``); barrier; grouped GEMM, SwiGLU + quantizer, grouped
    GEMM on the received buffer as it is; ``ks_moe_scatter_rows`` writes every result row back to
    the position the source's unpermute expects; barrier; weighted unpermute. The only host read
    (the number of received rows, for the row counts of the kernels in the middle) is issued
    right after the plan and waited for after the first GEMM has been enqueued.

    Buffers (``torch.distributed._symmetric_memory``) are sized for the worst case, every row of
    every rank landing on one rank. The returned tensor is overwritten by the next call.
    """

    def __init__(self, tokens_per_rank: int, top_k: int, hidden: int, inter: int, num_experts: int, group=None,
                 device=None):
        import torch.distributed._symmetric_memory as symm_mem
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.t_local, self.k, self.hidden, self.inter, self.num_experts = tokens_per_rank, top_k, hidden, inter, num_experts
        self.per = -(-num_experts // self.world)
        self.e_pad = self.per * self.world
        self.e_local = max(0, min(self.per, num_experts - self.rank * self.per))
        dev = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.dev = dev
        self.pairs = tokens_per_rank * top_k
        self.cap = self.pairs * self.world
        self.recv_q = symm_mem.empty((self.cap, hidden), dtype=torch.uint8, device=dev)
        self.recv_s = symm_mem.empty((self.cap, hidden // BLOCK), dtype=torch.float32, device=dev)
        self.back = symm_mem.empty((self.pairs, hidden), dtype=torch.bfloat16, device=dev)
        self.h_q = symm_mem.rendezvous(self.recv_q, self.group)
        self.h_s = symm_mem.rendezvous(self.recv_s, self.group)
        self.h_back = symm_mem.rendezvous(self.back, self.group)
        self.q_ptrs = [int(p) for p in self.h_q.buffer_ptrs]
        self.s_ptrs = [int(p) for p in self.h_s.buffer_ptrs]
        self.back_ptrs = [int(p) for p in self.h_back.buffer_ptrs]
        i32 = dict(dtype=torch.int32, device=dev)
        self.counts_all = torch.zeros(self.world, self.e_pad, **i32)
        self.counts_mine = torch.zeros(self.e_pad, **i32)
        self.dst_base = torch.zeros(self.e_pad, **i32)
        self.local_offsets = torch.zeros(self.per + 1, **i32)
        self.seg_start = torch.zeros(self.per * self.world + 1, **i32)
        self.ret_base = torch.zeros(self.per * self.world, **i32)
        self.total_host = torch.zeros(1, dtype=torch.int32).pin_memory()
        self.total_ready = torch.cuda.Event()
        # activations between the two GEMMs, worst case
        self.h = torch.empty(self.cap, 2 * inter, dtype=torch.bfloat16, device=dev)
        self.a8 = torch.empty(self.cap, inter, dtype=torch.float8_e4m3fn, device=dev)
        self.a_s = torch.empty(self.cap, inter // BLOCK, dtype=torch.float32, device=dev)
        self.y = torch.empty(self.cap, hidden, dtype=torch.bfloat16, device=dev)

    def __call__(self, tokens, topk_ids, topk_weights, w1_8, w1_s, w2_8, w2_s, ops=None):
        from . import activation, moe
        ops = ops or LibraryOps()
        k, hidden, inter = self.k, self.hidden, self.inter
        ids32 = topk_ids.to(device=self.dev, dtype=torch.int32).contiguous()
        weights = topk_weights.to(device=self.dev, dtype=torch.float32).contiguous()
        sorted_ids, offsets = ops.permutation(ids32, self.num_experts)
        self.counts_mine[:self.num_experts] = offsets[1:] - offsets[:-1]
        dist.all_gather_into_tensor(self.counts_all, self.counts_mine, group=self.group)
        moe.dispatch_plan(self.dst_base, self.local_offsets, self.seg_start, self.ret_base, self.counts_all,
                          self.world, self.rank, self.per)
        self.total_host.copy_(self.local_offsets[self.per:], non_blocking=True)
        self.total_ready.record()
        moe.permute_quant_fp8_scatter(self.q_ptrs, self.s_ptrs, self.cap, self.dst_base, offsets, self.num_experts,
                                      self.per, tokens, sorted_ids, self.t_local, k, hidden)
        self.h_q.barrier()    # every rank's rows (and scales) for my experts have landed
        if self.e_local > 0:
            moe.grouped_gemm_fp8_blockwise(self.h, self.recv_q.view(torch.float8_e4m3fn), w1_8, self.recv_s, w1_s,
                                           self.local_offsets, self.e_local, self.cap, 2 * inter, hidden, b_layout="nk")
        self.total_ready.synchronize()
        total = int(self.total_host[0])
        if self.e_local > 0 and total > 0:
            activation.swiglu_packed_quant_fp8(self.a8, self.a_s, self.h, total, inter)
            moe.grouped_gemm_fp8_blockwise(self.y, self.a8, w2_8, self.a_s, w2_s, self.local_offsets, self.e_local,
                                           self.cap, hidden, inter, b_layout="nk")
        moe.scatter_rows(self.back_ptrs, self.pairs, self.y, self.cap, self.seg_start, self.ret_base,
                         self.per * self.world, hidden)
        self.h_back.barrier()  # every expert's rows of my tokens are back
        return ops.unpermute(self.back, sorted_ids, weights, self.t_local, k)


def swiglu(gate_up: torch.Tensor) -> torch.Tensor:
    """silu(gate) * up for a [rows, 2*I] tensor holding gate then up."""
    i = gate_up.shape[1] // 2
    g = gate_up[:, :i].float()
    return (torch.nn.functional.silu(g) * gate_up[:, i:].float()).to(gate_up.dtype)


def expert_parallel_moe(tokens: torch.Tensor, topk_ids: torch.Tensor, topk_weights: torch.Tensor,
                        w1_8: torch.Tensor, w1_s: torch.Tensor, w2_8: torch.Tensor, w2_s: torch.Tensor,
                        num_experts: int, ops=None, group=None) -> torch.Tensor:
    """One MoE layer with experts split contiguously over the ranks.

    tokens [T_local, H] bf16 (this rank's tokens); topk_ids / topk_weights
    [T_local, k]; w1_8 [E_local, 2I, H] with w1_s [E_local, 2I/128, H/128];
    w2_8 [E_local, H, I] with w2_s [E_local, H/128, I/128] (this rank's experts,
    weights stored [N,K]). Steps, each one kernel (or one collective) on the
    tensors' device: counting-sort permutation of the (token, slot) pairs by
    expert -> gather fused with the 1 x 128 quantizer (rows travel as fp8 codes
    plus fp32 scales, half the bytes of bf16) -> exchange counts -> all-to-all
    to the experts' ranks -> regroup by local expert -> grouped FP8 GEMM
    (gate/up) -> SwiGLU fused with the re-quantisation -> grouped FP8 GEMM
    (down) -> all-to-all back -> weighted sum per token in pair order.
    With more than one rank the split sizes of the all-to-alls are read back to
    the host once (two small vectors); with one rank nothing leaves the device.
    Returns [T_local, H] bf16."""
    ops = ops or LibraryOps()
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    t_local, hidden = tokens.shape
    k = topk_ids.shape[1]
    dev = tokens.device
    ids32 = topk_ids.to(device=dev, dtype=torch.int32).contiguous()
    weights = topk_weights.to(device=dev, dtype=torch.float32).contiguous()
    sorted_ids, offsets = ops.permutation(ids32, num_experts)      # sorted by expert = by destination rank
    x8, x_s = ops.permute_quant(tokens, sorted_ids, k)
    inter2, inter = w1_8.shape[1], w2_8.shape[2]
    if world > 1:
        per = -(-num_experts // world)
        counts = (offsets[1:] - offsets[:-1]).to(torch.int64)
        recv_matrix = exchange_counts(counts, num_experts, world, group)
        pad = per * world - num_experts
        padded = torch.cat([counts, counts.new_zeros(pad)]) if pad else counts
        sizes = torch.stack([padded.view(world, per).sum(1), recv_matrix.sum(1)]).cpu()   # the one host read
        send_l, recv_l = sizes[0].tolist(), sizes[1].tolist()
        r8 = all_to_all_rows(x8.view(torch.uint8), send_l, recv_l, group).view(x8.dtype)
        r_s = all_to_all_rows(x_s, send_l, recv_l, group)
        perm, local_offsets = received_to_expert_major(recv_matrix, sum(recv_l))
        r8 = ops.gather_rows(r8, perm)
        r_s = ops.gather_rows(r_s, perm)
    else:
        r8, r_s, local_offsets = x8, x_s, offsets
    if r8.shape[0] > 0:
        h = ops.grouped_fp8_gemm(r8, w1_8, local_offsets, r_s, w1_s, inter2, hidden, "nk")
        a8, a_s = ops.swiglu_quant(h)
        y = ops.grouped_fp8_gemm(a8, w2_8, local_offsets, a_s, w2_s, hidden, inter, "nk")
    else:
        y = tokens.new_zeros((0, hidden))
    if world > 1:
        # undo the regrouping (the inverse of a permutation, on the device), then send every
        # row back to the rank its token lives on
        inverse = torch.empty_like(perm)
        inverse[perm.to(torch.int64)] = torch.arange(perm.numel(), dtype=perm.dtype, device=perm.device)
        y = all_to_all_rows(ops.gather_rows(y, inverse), recv_l, send_l, group)
    return ops.unpermute(y, sorted_ids, weights, t_local, k)
