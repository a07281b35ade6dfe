"""Generates tests/golden/int4_checkpoint.npz: small GPTQ and AWQ layers packed
by the packers of vLLM (``vllm.model_executor.layers.quantization.utils.
quant_utils``: ``gptq_pack``, ``awq_pack``, ``pack_cols``), the provider the
reference project routes its weight-repack op to
(``bindings/python/kernel_set/backends/_quant_ext.py:217-241``). The reference
itself holds no packer for these formats, so these vectors are what pins the
oracle's statement of them. Runs on the CPU; needs vLLM importable.
"""
from __future__ import annotations

import os

import numpy as np
import torch
from vllm.model_executor.layers.quantization.utils import quant_utils as vq

HERE = os.path.dirname(os.path.abspath(__file__))


def main():
    g = torch.Generator().manual_seed(20)
    k, n, gs = 256, 64, 64
    groups = k // gs
    codes = torch.randint(0, 16, (k, n), generator=g, dtype=torch.int32)
    zeros = torch.randint(1, 17, (groups, n), generator=g, dtype=torch.int32)     # 1..16: a first-version file stores zero-1
    zeros_awq = torch.randint(0, 16, (groups, n), generator=g, dtype=torch.int32)
    rand_perm = torch.randperm(k, generator=g)
    g_idx = (torch.arange(k, dtype=torch.int32) // gs)[rand_perm].contiguous()

    out = {
        "k": np.int64(k), "n": np.int64(n), "group_size": np.int64(gs),
        "codes": codes.numpy(), "zeros_gptq": zeros.numpy(), "zeros_awq": zeros_awq.numpy(),
        "gptq_qweight": vq.gptq_pack(codes, 4, k, n).numpy(),
        "gptq_qzeros_v1": vq.pack_cols(zeros - 1, 4, groups, n).numpy(),
        "gptq_qzeros_v2": vq.pack_cols(zeros_awq, 4, groups, n).numpy(),
        # activation order: the file holds the rows in the order the layer was quantised
        "act_order_rows": rand_perm.numpy(), "g_idx": g_idx.numpy(),
        "gptq_qweight_act_order": vq.gptq_pack(codes[rand_perm].contiguous(), 4, k, n).numpy(),
        "awq_qweight": vq.awq_pack(codes, 4, k, n).numpy(),
        "awq_qzeros": vq.awq_pack(zeros_awq, 4, groups, n).numpy(),
    }
    np.savez_compressed(os.path.join(HERE, "int4_checkpoint.npz"), **out)
    print("wrote int4_checkpoint.npz:", {k_: getattr(v, "shape", ()) for k_, v in out.items()})


if __name__ == "__main__":
    main()
