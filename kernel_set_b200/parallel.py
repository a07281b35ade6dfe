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


def plan_dispatch(expert_ids: torch.Tensor, num_experts: int, world: int):
    """For this rank's (token, slot) pairs: the order that sorts them by expert
    (stable), and how many go to each rank. ``expert_ids`` is [T, k]."""
    flat = expert_ids.reshape(-1).to(torch.int64)
    order = torch.sort(flat, stable=True).indices
    counts = torch.bincount(flat, minlength=num_experts)
    per = -(-num_experts // world)
    pad = per * world - num_experts
    if pad:
        counts = torch.cat([counts, counts.new_zeros(pad)])
    send_counts = counts.view(world, per).sum(1)
    return order, counts[:num_experts], send_counts


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


def received_to_expert_major(recv_counts_matrix: torch.Tensor):
    """Rows arrive grouped by source rank, and inside a source by local expert.
    Returns (perm, offsets): ``received[perm]`` is sorted by local expert (source
    rank order inside an expert), ``offsets`` int32 [E_local+1]."""
    world, per = recv_counts_matrix.shape
    counts = recv_counts_matrix.to(torch.int64)
    src_base = torch.zeros(world, per, dtype=torch.int64)
    flat = counts.reshape(-1)
    starts = torch.cumsum(flat, 0) - flat
    src_base = starts.view(world, per)
    idx: List[torch.Tensor] = []
    for e in range(per):
        for r in range(world):
            c = int(counts[r, e])
            if c:
                idx.append(torch.arange(c, dtype=torch.int64) + int(src_base[r, e]))
    perm = torch.cat(idx) if idx else torch.zeros(0, dtype=torch.int64)
    offsets = torch.zeros(per + 1, dtype=torch.int32)
    offsets[1:] = torch.cumsum(counts.sum(0), 0).to(torch.int32)
    return perm, offsets
