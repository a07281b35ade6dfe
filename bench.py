#!/usr/bin/env python3
"""Benchmark of the quantized-GEMM path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]

One "step" is one pass of the headline workload: the DeepSeek-V3-shaped FP8
block-scaled GEMM, A bf16 [4096, 7168] ~N(0,1) quantized in-path to e4m3 with
1 x 128 fp32 scales, times a resident e4m3 weight [N=7168, K=7168] with
128 x 128 fp32 block scales, bf16 output. Synthetic seeded tensors of that
shape stand in for model weights and activations. At N > 1 the weight is split
by N across the ranks (whole 128-column blocks, no collective) and every rank
multiplies the full activation with its shard: total work is fixed (strong
scaling).

Rank 0 prints ONE JSON line. `value` is 2*M*N*K*steps / device time of the
timed region (inputs resident in HBM, quantizer and GEMM both inside);
`roofline` describes the GEMM kernel alone; `e2e` repeats the measurement with
the activation starting in pinned host memory and the result read back;
`cpu_baseline` is the CPU oracle of the same step timed on this machine's
host cores. Further keys are secondary measurements of the same path:
`shape_7168` (the M=N=K=7168 target shape), `w4a16_decode` (the int4 decode
sweep), `competitors` (vLLM's CUTLASS block-scaled FP8 GEMM and Marlin on the
same inputs, where they load), `moe_layer` / `cfg4` (the MoE configuration) and
`cfg5` (the row-parallel configuration) with their parity checks.
`--impl reference` prints only the CPU measurement.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

M, N, K = 4096, 7168, 7168
WORKLOAD = "fp8_blockwise_gemm M=4096 N=7168 K=7168 (A bf16 quantized in-path 1x128; W e4m3 [N,K] 128x128 scales; bf16 out)"
ROTATE = 3  # input/output sets cycled so that no step finds its operands in L2


def parse_args():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=200)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--impl", default="b200", choices=["b200", "reference"])
    p.add_argument("--no-extras", action="store_true", help="skip every secondary measurement")
    p.add_argument("--m", type=int, default=M, help="rows of A (default: the headline 4096)")
    p.add_argument("--workload", default="cfg2", choices=["cfg2", "cfg4", "cfg5"],
                   help="cfg2: the headline line (default); cfg4 / cfg5: print only that configuration's record")
    return p.parse_args()


def config_of(m: int, world: int) -> dict:
    """The workload description; both arms print exactly this."""
    return {"workload": WORKLOAD, "m": m, "n": N, "k": K,
            "parallelism": "single GPU" if world == 1 else f"column-parallel by N over {world} GPUs, no collective",
            "l2": f"rotating {ROTATE} operand/output sets per rank, larger than L2 in total"}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_burst": float(d["bf16_tflops"]),
                "bf16_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "source": "measured"}
    except Exception:
        return {"hbm_gbs": 6650.0, "bf16_burst": 1590.0, "bf16_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [x.strip() for x in ln.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                smax.append(float(parts[1]))
            except ValueError:
                continue
            for nm, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def make_inputs(m: int):
    """Seeded CPU tensors of the headline shape; the weight is block-quantized
    once with the oracle's statement of the reference's input preparation."""
    import torch
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import ks_oracle as orc
    g = torch.Generator().manual_seed(0)
    a = torch.randn(m, K, generator=g).to(torch.bfloat16)
    w_nk = torch.randn(N, K, generator=g) * 0.02
    # quantize_weight_blocks works on [K,N]; a transposed view gives [N,K] blocks
    b8_kn, bs_kn = orc.quantize_weight_blocks(w_nk.t(), 128, 128)
    return a, b8_kn.t().contiguous(), bs_kn.t().contiguous()


def cpu_step_seconds(a, b8_nk, bs_nk, budget_s: float = 20.0):
    """The oracle's statement of one step on the host cores: group quantizer,
    operand dequantisation, fp32 matmul, bf16 rounding."""
    import torch
    import ks_oracle as orc

    def step():
        a8, a_s = orc.quantize_fp8_group(a, 128)
        return orc.fp8_gemm_blockwise(a8, b8_nk, a_s, bs_nk, layout="nk", out_dtype=torch.bfloat16)

    step()
    times = []
    t_end = time.perf_counter() + budget_s
    while len(times) < 3 or (time.perf_counter() < t_end and len(times) < 10):
        t0 = time.perf_counter()
        step()
        times.append(time.perf_counter() - t0)
        if time.perf_counter() > t_end and len(times) >= 2:
            break
    return statistics.median(times), len(times), torch.get_num_threads()


def run_reference(args):
    """CPU arm: the reference's torch statement of the step (restated in
    oracle/ks_oracle.py) on ALL of this machine's host cores. Rank 0 only; under
    a launcher that pins OMP_NUM_THREADS=1 the thread count is set back."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import torch
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    a, b8, bs = make_inputs(args.m)
    import ks_oracle as orc

    def step():
        a8, a_s = orc.quantize_fp8_group(a, 128)
        return orc.fp8_gemm_blockwise(a8, b8, a_s, bs, layout="nk", out_dtype=torch.bfloat16)

    for _ in range(max(1, min(args.warmup, 2))):
        step()
    steps = max(1, min(args.steps, 5))
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / steps
    flops = 2.0 * args.m * N * K
    val = flops / dt / 1e12
    threads = torch.get_num_threads()
    line = {
        "impl": "reference", "metric": "fp8_blockwise_gemm_tflops", "value": val, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": min(args.warmup, 2), "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "fp8_e4m3",
        "data": "synthetic", "config": config_of(args.m, args.gpus),
        "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                         "sample": f"the whole step (quantizer + dequant + fp32 matmul), {steps} timed runs"},
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------
# device-side input preparation (the reference's recipes written with tensor ops)
# ---------------------------------------------------------------------------------
def block_quant_nk_device(w_nk):
    """128 x 128 block quantization of a [N,K] fp32 weight on its own device: the
    reference's input preparation (benchmarks/bench.py:1447-1461) written with
    tensor ops. Returns (e4m3 [N,K], scales [N/128, K/128])."""
    import torch
    n, k = w_nk.shape
    blocks = w_nk.view(n // 128, 128, k // 128, 128)
    scale = (blocks.abs().amax(dim=(1, 3)) / 448.0).clamp_min(1e-12)
    q = (blocks / scale[:, None, :, None]).to(torch.float8_e4m3fn).view(n, k)
    return q, scale.contiguous()


def fp8_launches(m: int, n: int, k: int, sms: int) -> int:
    """Kernels one ks_gemm_fp8_blockwise call launches (mirrors the tile choice of
    csrc/sm100_fp8_gemm.cu: a second kernel sums the K-parts of a split last round)."""
    tm = -(-m // 128)
    t256, t128 = tm * -(-n // 256), tm * -(-n // 128)
    bn = 256 if -(-t256 // sms) * 850 <= -(-t128 // sms) * 550 else 128
    tiles = t256 if bn == 256 else t128
    grid = min(tiles, sms)
    if tiles > grid and tiles % grid:
        s = min(8, grid // (tiles % grid))
        while s > 1 and -(-k // 128) // s < 4:
            s -= 1
        if s >= 2:
            return 2
    return 1


def timed(fn, steps, warmup, barrier, torch):
    for _ in range(warmup):
        fn()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    barrier()
    return e0.elapsed_time(e1) / steps


def median_us(fns, torch, reps=30, trials=3):
    """Median over trials of the mean device time of `reps` calls cycling through fns."""
    for f in fns:
        f()
    torch.cuda.synchronize()
    ts = []
    for _ in range(trials):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(reps):
            fns[i % len(fns)]()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1) * 1e3 / reps)
    return statistics.median(ts)


# ---------------------------------------------------------------------------------
# secondary measurements, 1 GPU
# ---------------------------------------------------------------------------------
def w4a16_decode_sweep(ks, torch, dev, peaks):
    """W4A16 decode shapes: achieved algorithmic GB/s. Three clocks per entry: `us` = device
    time per launch with the launches queued behind a spin kernel (the kernel alone);
    `us_back_to_back` = CUDA events around a plain host loop of calls; `host_us_per_call` =
    what one call costs the calling thread."""
    res = []
    for (k, n) in ((4096, 28672), (14336, 4096)):
        g = torch.Generator().manual_seed(1)
        copies = 3
        bps = [torch.randint(0, 256, (k // 2, n), generator=g, dtype=torch.uint8).to(dev) for _ in range(copies)]
        scales = (torch.randn(k // 128, n, generator=g).mul(0.02).abs() + 1e-3).to(torch.bfloat16).to(dev)
        zeros = torch.full((k // 128, n), 8.0, dtype=torch.bfloat16, device=dev)
        for m in (1, 8, 32, 128):
            a = torch.randn(m, k, generator=g).to(torch.bfloat16).to(dev)
            c = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
            iters = 24

            def call(i):
                ks.gemm.gemm_w4a16(c, a, bps[i % copies], scales, zeros, m, n, k, 128)

            for i in range(3):
                call(i)
            torch.cuda.synchronize()
            queued, plain, host = [], [], []
            for _ in range(3):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                torch.cuda._sleep(6_000_000)
                e0.record()
                for i in range(iters):
                    call(i)
                e1.record()
                torch.cuda.synchronize()
                queued.append(e0.elapsed_time(e1) * 1e3 / iters)
                e0.record()
                t0 = time.perf_counter()
                for i in range(iters):
                    call(i)
                host.append((time.perf_counter() - t0) * 1e6 / iters)
                e1.record()
                torch.cuda.synchronize()
                plain.append(e0.elapsed_time(e1) * 1e3 / iters)
            us = statistics.median(queued)
            nbytes = k * n // 2 + 2 * (k // 128) * n * 2 + m * k * 2 + m * n * 2
            gbs = nbytes / (us * 1e-6) / 1e9
            res.append({"m": m, "k": k, "n": n, "us": round(us, 2), "gbs": round(gbs, 1),
                        "frac_of_measured_hbm": round(gbs / peaks["hbm_gbs"], 4),
                        "frac_of_nominal_8000": round(gbs / 8000.0, 4),
                        "us_back_to_back": round(statistics.median(plain), 2),
                        "host_us_per_call": round(statistics.median(host), 2),
                        "tflops": round(2.0 * m * n * k / (us * 1e-6) / 1e12, 2)})
        del bps
    return res


def shape_7168(ks, torch, dev, peaks):
    """The target shape of the benchmark definition, M = N = K = 7168: GEMM alone, device inputs."""
    m = n = k = 7168
    g = torch.Generator(device=dev).manual_seed(3)
    sets = []
    for _ in range(2):
        a8 = torch.randn(m, k, generator=g, device=dev).clamp_(-3, 3).mul_(100).to(torch.float8_e4m3fn)
        a_s = torch.rand(m, k // 128, generator=g, device=dev) * 0.01 + 0.005
        b8, b_s = block_quant_nk_device(torch.randn(n, k, generator=g, device=dev) * 0.02)
        sets.append((a8, a_s, b8, b_s, torch.empty(m, n, dtype=torch.bfloat16, device=dev)))
    fns = [lambda i=i: ks.gemm.gemm_fp8_blockwise(sets[i][4], sets[i][0], sets[i][2], sets[i][1], sets[i][3], m, n, k,
                                                  b_layout="nk") for i in range(2)]
    us = median_us(fns, torch, reps=20)
    tf = 2.0 * m * n * k / (us * 1e-6) / 1e12
    return {"m": m, "n": n, "k": k, "us": round(us, 1), "tflops": round(tf, 1),
            "frac_of_2x_measured_bf16_burst": round(tf / (2 * peaks["bf16_burst"]), 4),
            "frac_of_nominal_4500": round(tf / 4500.0, 4)}


def competitor_rows(ks, torch, dev):
    """The Blackwell kernels the reference can route to, on this box, same inputs, same clock
    (CUDA events around rotating calls): vLLM's CUTLASS block-scaled FP8 GEMM on the headline
    and target shapes, Marlin on the decode shapes. Each row carries the relative Frobenius
    difference between the competitor's output and this library's on the same inputs."""
    rows = []
    try:
        from vllm import _custom_ops as ops
    except Exception as exc:
        return [{"provider": "vllm", "unavailable on this box": f"{type(exc).__name__}: {str(exc)[:200]}"}]
    # --- FP8 block-scaled GEMM ---
    for (m, n, k) in ((4096, 7168, 7168), (7168, 7168, 7168)):
        try:
            g = torch.Generator(device=dev).manual_seed(1)
            sets = []
            for _ in range(3):
                a = torch.randn(m, k, generator=g, device=dev).to(torch.bfloat16)
                a8 = torch.empty(m, k, dtype=torch.float8_e4m3fn, device=dev)
                a_s = torch.empty(m, k // 128, dtype=torch.float32, device=dev)
                ks.quant.quantize_fp8_group(a8, a_s, a, m, k, 128)
                b8, b_s = block_quant_nk_device(torch.randn(n, k, generator=g, device=dev) * 0.02)
                sets.append((a8, a_s, a_s.t().contiguous().t(), b8, b_s))
            outs = [torch.empty(m, n, dtype=torch.bfloat16, device=dev) for _ in range(3)]
            ours = [lambda i=i: ks.gemm.gemm_fp8_blockwise(outs[i], sets[i][0], sets[i][3], sets[i][1], sets[i][4], m, n,
                                                           k, b_layout="nk") for i in range(3)]
            theirs = [lambda i=i: ops.cutlass_scaled_mm(sets[i][0], sets[i][3].t(), sets[i][2], sets[i][4].t(),
                                                        torch.bfloat16) for i in range(3)]
            t_ours = median_us(ours, torch)
            o = theirs[0]()
            torch.cuda.synchronize()
            rel = float((o.float() - outs[0].float()).norm() / outs[0].float().norm())
            t_theirs = median_us(theirs, torch)
            rows.append({"op": "fp8_blockwise_gemm", "provider": "vllm cutlass_scaled_mm (1x128 / 128x128 fp32 scales)",
                         "m": m, "n": n, "k": k, "us": round(t_theirs, 1),
                         "tflops": round(2.0 * m * n * k / t_theirs / 1e6, 1), "ours_us": round(t_ours, 1),
                         "ours_tflops": round(2.0 * m * n * k / t_ours / 1e6, 1),
                         "rel_frobenius_vs_ours": rel})
            del sets, outs
        except Exception as exc:
            rows.append({"op": "fp8_blockwise_gemm", "provider": "vllm cutlass_scaled_mm", "m": m, "n": n, "k": k,
                         "unavailable on this box": f"{type(exc).__name__}: {str(exc)[:200]}"})
    # --- W4A16 ---
    try:
        from vllm.scalar_type import scalar_types
        from vllm.model_executor.layers.quantization.utils.marlin_utils import (marlin_make_workspace_new,
                                                                                marlin_permute_scales)
        import ks_oracle as orc
        for (k, n) in ((4096, 28672), (14336, 4096)):
            g = torch.Generator().manual_seed(2)
            codes = torch.randint(0, 16, (k, n), generator=g).to(torch.int32)
            scales = (torch.randn(k // 128, n, generator=g).mul(0.02).abs() + 1e-3).to(torch.bfloat16)
            words = orc.pack_int4_words(codes).to(dev)            # GPTQ packing: int32 [K/8, N]
            bp = orc.pack_int4_bytes(codes).to(dev)
            sc_d = scales.to(dev)
            zp_d = torch.full((k // 128, n), 8.0, dtype=torch.bfloat16, device=dev)
            empty = torch.empty(0, dtype=torch.int, device=dev)
            wq = [ops.gptq_marlin_repack(words.clone(), empty, k, n, 4) for _ in range(3)]
            ms = marlin_permute_scales(sc_d, k, n, 128)
            ws = marlin_make_workspace_new(dev)
            bps = [bp.clone() for _ in range(3)]
            for m in (1, 8, 32, 128):
                a = torch.randn(m, k, generator=g).to(torch.bfloat16).to(dev)
                c = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
                ours = [lambda i=i: ks.gemm.gemm_w4a16(c, a, bps[i], sc_d, zp_d, m, n, k, 128) for i in range(3)]
                theirs = [lambda i=i: ops.marlin_gemm(a, None, wq[i], None, ms, None, None, None, empty, empty, ws,
                                                      scalar_types.uint4b8, m, n, k, True, False, True, False)
                          for i in range(3)]
                o = theirs[0]()
                ours[0]()
                torch.cuda.synchronize()
                rel = float((o.float() - c.float()).norm() / c.float().norm())
                t_m, t_o = median_us(theirs, torch, 40), median_us(ours, torch, 40)
                nbytes = k * n // 2 + 2 * (k // 128) * n * 2 + m * k * 2 + m * n * 2
                rows.append({"op": "w4a16", "provider": "vllm marlin_gemm (gptq_marlin_repack, uint4b8, group 128)",
                             "m": m, "k": k, "n": n, "us": round(t_m, 2), "gbs": round(nbytes / t_m / 1e3, 1),
                             "ours_us": round(t_o, 2), "ours_gbs": round(nbytes / t_o / 1e3, 1),
                             "rel_frobenius_vs_ours": rel,
                             "clock": "back-to-back launches from the host loop, both sides"})
            del wq, bps
    except Exception as exc:
        rows.append({"op": "w4a16", "provider": "vllm marlin_gemm",
                     "unavailable on this box": f"{type(exc).__name__}: {str(exc)[:200]}"})
    return rows


# ---------------------------------------------------------------------------------
# the sharded configurations
# ---------------------------------------------------------------------------------
def run_cfg5(args, torch, dist, ks, parallel, dev, rank, world):
    """Row-parallel GEMM: A bf16 [16384, 28672], W e4m3 [8192, 28672], K split over the
    ranks, bf16 partial outputs all-reduced. GEMM and all-reduce are timed separately; rank 0
    checks a 256 x 256 window of the reduced result against the oracle on the unsplit operands."""
    import ks_oracle as orc
    m5, n5, k5 = 16384, 8192, 28672
    lo, hi = parallel.block_range(k5, rank, world)
    g = torch.Generator(device=dev).manual_seed(1234 + rank)
    a_sh = torch.randn(m5, hi - lo, generator=g, device=dev).to(torch.bfloat16)
    w8, ws = block_quant_nk_device(torch.randn(n5, hi - lo, generator=g, device=dev) * 0.02)
    a8 = torch.empty(m5, hi - lo, dtype=torch.float8_e4m3fn, device=dev)
    a_s = torch.empty(m5, (hi - lo) // 128, dtype=torch.float32, device=dev)
    out = torch.empty(m5, n5, dtype=torch.bfloat16, device=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def quant():
        ks.quant.quantize_fp8_group(a8, a_s, a_sh, m5, hi - lo, 128)

    def gemm():
        ks.gemm.gemm_fp8_blockwise(out, a8, w8, a_s, ws, m5, n5, hi - lo, b_layout="nk")

    def reduce():
        if world > 1:
            dist.all_reduce(out)

    def step():
        quant(); gemm(); reduce()

    # parity first: one step, then a window of the result against the oracle
    step()
    barrier()
    win = 256
    pieces = [a8[:win].view(torch.uint8).contiguous(), a_s[:win].contiguous(),
              w8[:win].view(torch.uint8).contiguous(), ws[:win // 128].contiguous()]
    gathered = []
    for t in pieces:
        if world > 1:
            # K-shards may differ by one block between ranks: pad to the widest before gathering
            width = torch.tensor([t.shape[1]], device=dev)
            widths = [torch.zeros_like(width) for _ in range(world)]
            dist.all_gather(widths, width)
            wmax = int(max(int(w) for w in widths))
            padded = torch.zeros(t.shape[0], wmax, dtype=t.dtype, device=dev)
            padded[:, :t.shape[1]] = t
            parts = [torch.empty_like(padded) for _ in range(world)]
            dist.all_gather(parts, padded)
            gathered.append(torch.cat([p[:, :int(w)] for p, w in zip(parts, widths)], dim=1).cpu())
        else:
            gathered.append(t.cpu())
    parity, ref32 = None, None
    if rank == 0:
        a8w, asw, w8w, wsw = gathered
        ref32 = orc.fp8_gemm_blockwise(a8w.view(torch.float8_e4m3fn), w8w.view(torch.float8_e4m3fn), asw, wsw, 128, 128,
                                       "nk", out_dtype=None)
        got = out[:win, :win].float().cpu()
        err_ulp = ((got - ref32).abs() / orc.bf16_ulp(ref32).float())
        parity = {"window": f"rows 0..{win}, columns 0..{win} of the all-reduced output vs the oracle on unsplit K",
                  "rel_frobenius": orc.rel_frobenius(got, ref32.to(torch.bfloat16).float()),
                  "max_err_bf16_ulp": float(err_ulp.max()), "frac_above_2_ulp": float((err_ulp > 2).float().mean()),
                  "note": "bf16 partials are rounded once per rank before the sum and once after"}

    steps = max(3, min(args.steps, 10))
    ms_step = timed(step, steps, 2, barrier, torch)
    ms_quant = timed(quant, steps, 1, barrier, torch)
    ms_gemm = timed(gemm, steps, 1, barrier, torch)
    ms_red = timed(reduce, steps, 1, barrier, torch) if world > 1 else 0.0

    # the same step with fp32 partials: twice the bytes on NVLink, one rounding in all
    fp32 = None
    if world > 1:
        out32 = torch.empty(m5, n5, dtype=torch.float32, device=dev)

        def step32():
            quant()
            ks.gemm.gemm_fp8_blockwise(out32, a8, w8, a_s, ws, m5, n5, hi - lo, b_layout="nk")
            dist.all_reduce(out32)

        step32()
        barrier()
        par32 = None
        if rank == 0:
            got32 = out32[:win, :win].to(torch.bfloat16).float().cpu()
            e32 = ((got32 - ref32).abs() / orc.bf16_ulp(ref32).float())
            par32 = {"rel_frobenius": orc.rel_frobenius(got32, ref32.to(torch.bfloat16).float()),
                     "max_err_bf16_ulp": float(e32.max()), "frac_above_2_ulp": float((e32 > 2).float().mean())}
        ms_step32 = timed(step32, steps, 1, barrier, torch)
        ms_red32 = timed(lambda: dist.all_reduce(out32), steps, 1, barrier, torch)
        t32 = torch.tensor([ms_step32, ms_red32], dtype=torch.float64, device=dev)
        dist.all_reduce(t32, op=dist.ReduceOp.MAX)
        fp32 = {"ms_per_step": float(t32[0]), "allreduce_us": float(t32[1]) * 1e3,
                "value": 2.0 * m5 * n5 * k5 / (float(t32[0]) * 1e-3) / 1e12, "parity": par32}
        del out32
    # the all-reduce fused with the GEMM over peer memory: every rank's epilogue stores its
    # partial of a row block into the owner's memory, the owner adds the slots in fp32 and
    # writes the rows into every rank's output (kernel_set_b200.parallel.FusedRowParallel)
    fused = None
    if world > 1:
        try:
            fused = {}
            for tag, pdt in (("fp32_slots", torch.float32), ("bf16_slots", torch.bfloat16)):
                layer = parallel.FusedRowParallel(m5, n5, part_dtype=pdt, device=dev)

                def step_fused():
                    quant()
                    layer.multiply(a8, a_s, w8, ws)

                def reduce_scatter_only():
                    quant()
                    layer.multiply(a8, a_s, w8, ws, gather=False)

                res = layer.multiply(a8, a_s, w8, ws)
                barrier()
                parf = None
                if rank == 0:
                    gotf = res[:win, :win].float().cpu()
                    ef = ((gotf - ref32).abs() / orc.bf16_ulp(ref32).float())
                    parf = {"rel_frobenius": orc.rel_frobenius(gotf, ref32.to(torch.bfloat16).float()),
                            "max_err_bf16_ulp": float(ef.max()), "frac_above_2_ulp": float((ef > 2).float().mean())}
                tf = torch.tensor([timed(step_fused, steps, 1, barrier, torch), timed(reduce_scatter_only, steps, 1, barrier, torch)],
                                  dtype=torch.float64, device=dev)
                dist.all_reduce(tf, op=dist.ReduceOp.MAX)
                fused[tag] = {"ms_per_step": float(tf[0]), "value": 2.0 * m5 * n5 * k5 / (float(tf[0]) * 1e-3) / 1e12,
                              "ms_per_step_reduce_scatter_only": float(tf[1]), "parity": parf}
                del layer, res
                torch.cuda.empty_cache()
        except Exception as exc:   # symmetric memory not available on this machine
            fused = {"unavailable": f"{type(exc).__name__}: {exc}"[:300]}
    t = torch.tensor([ms_step, ms_quant, ms_gemm, ms_red], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step, ms_quant, ms_gemm, ms_red = [float(v) for v in t.tolist()]
    flops = 2.0 * m5 * n5 * k5
    ring_bytes = 2.0 * (world - 1) / world * m5 * n5 * 2
    del a_sh, w8, a8, out
    torch.cuda.empty_cache()
    return {
        "metric": "fp8_blockwise_gemm_tflops", "value": flops / (ms_step * 1e-3) / 1e12, "unit": "TFLOP/s",
        "n_gpus": world, "steps": steps, "ms_per_step": ms_step, "scaling": "strong",
        "config": {"workload": "row-parallel fp8_blockwise_gemm M=16384 N=8192 K=28672, K split, bf16 all-reduce",
                   "k_per_gpu": hi - lo, "l2": "operands (0.7 GB per rank at 8 GPUs, 2 GB at 1) exceed L2"},
        "gemm_us": ms_gemm * 1e3, "quantizer_us": ms_quant * 1e3, "allreduce_us": ms_red * 1e3,
        "gemm_tflops_per_gpu": flops / world / (ms_gemm * 1e-3) / 1e12,
        "allreduce_busbw_gbs": (ring_bytes / (ms_red * 1e-3) / 1e9) if world > 1 else None,
        "parity": parity, "fp32_partials": fp32, "fused_over_peer_memory": fused}


def moe_small_parity(torch, dist, ks, parallel, dev, rank, world):
    """The expert-parallel layer on a reduced configuration (256 tokens, hidden 512, 32 experts,
    intermediate 256, top-4), through the same kernels and collectives as the full one; every
    rank builds the same seeded problem and rank 0 compares its tokens with a dense,
    token-by-token oracle evaluation."""
    import ks_oracle as orc
    tokens, hidden, experts, inter, topk = 256, 512, 32, 256, 4
    g = torch.Generator().manual_seed(4)
    x = torch.randn(tokens, hidden, generator=g).to(torch.bfloat16)
    w, ids = orc.moe_route(torch.randn(tokens, experts, generator=g), topk)
    w1, s1, w2, s2 = [], [], [], []
    for _ in range(experts):
        q, s = orc.quantize_weight_blocks((torch.randn(2 * inter, hidden, generator=g) * 0.05).t())
        w1.append(q.t().contiguous()); s1.append(s.t().contiguous())
        q, s = orc.quantize_weight_blocks((torch.randn(hidden, inter, generator=g) * 0.05).t())
        w2.append(q.t().contiguous()); s2.append(s.t().contiguous())
    w1, s1, w2, s2 = torch.stack(w1), torch.stack(s1), torch.stack(w2), torch.stack(s2)
    t_local = tokens // world
    sl = slice(rank * t_local, (rank + 1) * t_local)
    e_lo, e_hi = parallel.expert_range(experts, rank, world)
    got = parallel.expert_parallel_moe(x[sl].to(dev), ids[sl].to(dev), w[sl].to(dev), w1[e_lo:e_hi].to(dev),
                                       s1[e_lo:e_hi].to(dev), w2[e_lo:e_hi].to(dev), s2[e_lo:e_hi].to(dev), experts)
    torch.cuda.synchronize()
    if rank != 0:
        return None
    ref = torch.zeros(t_local, hidden, dtype=torch.float32)
    for t in range(t_local):
        x8, xs = orc.quantize_fp8_group(x[t:t + 1], 128)
        for slot in range(topk):
            e = int(ids[t, slot])
            h = orc.fp8_gemm_blockwise(x8, w1[e], xs, s1[e], layout="nk")
            a8, a_s = orc.quantize_fp8_group(orc.swiglu_packed(h), 128)
            ref[t] += float(w[t, slot]) * orc.fp8_gemm_blockwise(a8, w2[e], a_s, s2[e], layout="nk")[0].float()
    return {"config": "256 tokens, hidden 512, 32 experts, inter 256, top-4; rank 0's tokens vs a dense oracle evaluation",
            "rel_frobenius": orc.rel_frobenius(got.float().cpu(), ref)}


def run_cfg4(args, torch, dist, ks, parallel, dev, rank, world):
    """MoE layer, DeepSeek-V3 sizes: 4096 tokens, hidden 7168, 256 experts, intermediate 2048,
    top-8. Experts are split contiguously over the ranks, tokens evenly; dispatch and combine
    are all-to-alls. Weights are generated and block-quantized on the device, one expert at a
    time; routing comes from the gate kernel on seeded logits."""
    tokens, hidden, experts, inter, topk = 4096, 7168, 256, 2048, 8
    parity = moe_small_parity(torch, dist, ks, parallel, dev, rank, world)
    e_lo, e_hi = parallel.expert_range(experts, rank, world)
    e_local = e_hi - e_lo
    g = torch.Generator(device=dev).manual_seed(99 + rank)
    w1 = torch.empty(e_local, 2 * inter, hidden, dtype=torch.float8_e4m3fn, device=dev)
    s1 = torch.empty(e_local, 2 * inter // 128, hidden // 128, dtype=torch.float32, device=dev)
    w2 = torch.empty(e_local, hidden, inter, dtype=torch.float8_e4m3fn, device=dev)
    s2 = torch.empty(e_local, hidden // 128, inter // 128, dtype=torch.float32, device=dev)
    for e in range(e_local):
        w1[e], s1[e] = block_quant_nk_device(torch.randn(2 * inter, hidden, generator=g, device=dev) * 0.02)
        w2[e], s2[e] = block_quant_nk_device(torch.randn(hidden, inter, generator=g, device=dev) * 0.02)
    t_local = tokens // world
    gt = torch.Generator().manual_seed(7)  # logits and tokens are global and identical on every rank
    logits = torch.randn(tokens, experts, generator=gt)
    x = torch.randn(tokens, hidden, generator=gt).to(torch.bfloat16)
    sl = slice(rank * t_local, (rank + 1) * t_local)
    x_l, logits_l = x[sl].to(dev), logits[sl].to(dev)
    w_l = torch.empty(t_local, topk, dtype=torch.float32, device=dev)
    ids_l = torch.empty(t_local, topk, dtype=torch.int32, device=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def step():
        ks.moe.gate_softmax_topk(w_l, ids_l, logits_l, t_local, experts, topk, renormalize=True)
        return parallel.expert_parallel_moe(x_l, ids_l, w_l, w1, s1, w2, s2, experts)

    steps = max(3, min(args.steps, 10))
    ms_step = timed(step, steps, 2, barrier, torch)
    # the same layer with dispatch and combine as peer stores (FusedExpertParallel)
    fused = None
    if world > 1:
        try:
            layer = parallel.FusedExpertParallel(t_local, topk, hidden, inter, experts, device=dev)

            def step_fused():
                ks.moe.gate_softmax_topk(w_l, ids_l, logits_l, t_local, experts, topk, renormalize=True)
                return layer(x_l, ids_l, w_l, w1, s1, w2, s2)

            same = bool(torch.equal(step_fused(), step()))
            ms_fused = timed(step_fused, steps, 2, barrier, torch)
            tf = torch.tensor([ms_fused, 0.0 if same else 1.0], dtype=torch.float64, device=dev)
            dist.all_reduce(tf, op=dist.ReduceOp.MAX)
            fused = {"ms_per_step": float(tf[0]), "equal_to_the_nccl_path_bit_for_bit": float(tf[1]) == 0.0}
            del layer
            torch.cuda.empty_cache()
        except Exception as exc:   # symmetric memory not available on this machine
            fused = {"unavailable": f"{type(exc).__name__}: {exc}"[:300]}
    # the two grouped GEMMs alone, on the rows this rank's experts receive
    import ks_oracle as orc
    _, ids_all = orc.moe_route(logits, topk)
    counts = torch.bincount(ids_all.reshape(-1), minlength=experts)[e_lo:e_hi]
    offs = torch.zeros(e_local + 1, dtype=torch.int32)
    offs[1:] = torch.cumsum(counts, 0).to(torch.int32)
    rows = int(offs[-1])
    offs_d = offs.to(dev)
    xa8, xas = ks.dispatch.per_token_group_quant(torch.randn(rows, hidden, generator=g, device=dev).to(torch.bfloat16))
    ha8, has = ks.dispatch.per_token_group_quant(torch.randn(rows, inter, generator=g, device=dev).to(torch.bfloat16))

    def gemms():
        ks.dispatch.moe(xa8, w1, offs_d, n=2 * inter, k=hidden, a_scale=xas, b_scale=s1, b_layout="nk")
        ks.dispatch.moe(ha8, w2, offs_d, n=hidden, k=inter, a_scale=has, b_scale=s2, b_layout="nk")

    ms_gemm = timed(gemms, steps, 2, barrier, torch)
    t = torch.tensor([ms_step, ms_gemm, float(rows)], dtype=torch.float64, device=dev)
    if world > 1:
        tmax = t.clone()
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        ms_step, ms_gemm, rows_all = float(tmax[0]), float(tmax[1]), float(t[2])
    else:
        ms_step, ms_gemm, rows_all = float(t[0]), float(t[1]), float(t[2])
    flops = 2.0 * rows_all * (2 * inter * hidden + hidden * inter)
    weight_bytes = e_local * (2 * inter * hidden + hidden * inter)
    del w1, w2
    torch.cuda.empty_cache()
    return {
        "metric": "moe_grouped_fp8_gemm_tflops", "value": flops / (ms_step * 1e-3) / 1e12, "unit": "TFLOP/s",
        "n_gpus": world, "steps": steps, "ms_per_step": ms_step, "scaling": "strong",
        "config": {"workload": "MoE layer, FP8 block-scaled: 4096 tokens, hidden 7168, 256 experts, inter 2048, top-8; "
                               "gate, permutation, fused gather+quant, all-to-all, grouped GEMM, fused SwiGLU+quant, "
                               "grouped GEMM, all-to-all, weighted unpermute",
                   "experts_per_gpu": e_local, "routed_rows": rows_all,
                   "l2": f"{weight_bytes / 1e9:.2f} GB of expert weights per rank, far larger than L2"},
        "grouped_gemms_us": ms_gemm * 1e3, "other_us": (ms_step - ms_gemm) * 1e3,
        "grouped_gemms_tflops_per_gpu": flops / world / (ms_gemm * 1e-3) / 1e12,
        "grouped_gemms_weight_gbs": weight_bytes / (ms_gemm * 1e-3) / 1e9,
        "parity": parity, "fused_over_peer_memory": fused}


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference(args)
        return

    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; the library has no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import kernel_set_b200 as ks
    from kernel_set_b200 import parallel

    if args.workload != "cfg2":
        rec = (run_cfg5 if args.workload == "cfg5" else run_cfg4)(args, torch, dist, ks, parallel, dev, rank, world)
        if rank == 0:
            print(json.dumps(rec), flush=True)
        if world > 1:
            dist.destroy_process_group()
        return

    peaks = measured_peaks()
    m = args.m
    a_cpu, b8_cpu, bs_cpu = make_inputs(m)
    b8_sh, bs_sh, (n_lo, n_hi) = parallel.shard_weight_columns(b8_cpu, bs_cpu, rank, world, "nk")
    n_local = n_hi - n_lo

    # ROTATE resident copies of every operand and output (> L2 in total)
    a_dev = [a_cpu.to(dev) for _ in range(ROTATE)]
    b_dev = [b8_sh.to(dev) for _ in range(ROTATE)]
    bs_dev = bs_sh.to(dev)
    a8 = [torch.empty(m, K, dtype=torch.float8_e4m3fn, device=dev) for _ in range(ROTATE)]
    a_s = [torch.empty(m, K // 128, dtype=torch.float32, device=dev) for _ in range(ROTATE)]
    out = [torch.empty(m, n_local, dtype=torch.bfloat16, device=dev) for _ in range(ROTATE)]
    a_pinned = a_cpu.pin_memory()
    out_pinned = torch.empty(m, n_local, dtype=torch.bfloat16).pin_memory()

    def quant(i):
        ks.quant.quantize_fp8_group(a8[i], a_s[i], a_dev[i], m, K, 128)

    def gemm(i):
        ks.gemm.gemm_fp8_blockwise(out[i], a8[i], b_dev[i], a_s[i], bs_dev, m, n_local, K, b_layout="nk")

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(max(args.warmup, 3)):
        quant(i % ROTATE)
        gemm(i % ROTATE)
    barrier()
    ks.runtime.stream_synchronize(0)

    # ---------------- timed region: resident inputs ----------------
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.25)
    gemm_events = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
                   for _ in range(args.steps)]
    quant_events = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    barrier()
    t_start, t_stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_start.record()
    for s in range(args.steps):
        i = s % ROTATE
        quant_events[s].record()
        quant(i)
        gemm_events[s][0].record()
        gemm(i)
        gemm_events[s][1].record()
    t_stop.record()
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    elapsed_ms = t_start.elapsed_time(t_stop)
    gemm_ms = statistics.mean(e0.elapsed_time(e1) for e0, e1 in gemm_events)
    quant_ms = statistics.mean(q.elapsed_time(g0) for q, (g0, _) in zip(quant_events, gemm_events))

    # ---------------- end to end: host activation in, host result out ----------------
    # Every step brings its activation in from pinned host memory, quantizes, multiplies and
    # copies the result back to pinned host memory. With several ranks each rank copies only
    # its 1/N of the rows over PCIe and the ranks exchange the slices over NVLink (NCCL
    # all-gather), instead of every rank pulling the whole activation through its own PCIe
    # link. The phases run on three streams over the three rotating buffer sets, so the
    # copy-in of step s+1 and the copy-out of step s-1 overlap the kernels of step s; events
    # carry the dependencies, including buffer reuse three steps later.
    s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    s_main = torch.cuda.current_stream()
    gather_rows = world > 1 and m % world == 0
    r_lo, r_hi = (rank * (m // world), (rank + 1) * (m // world)) if gather_rows else (0, m)
    a_pinned_mine = a_pinned[r_lo:r_hi]
    a_slice = [torch.empty(r_hi - r_lo, K, dtype=torch.bfloat16, device=dev) for _ in range(ROTATE)] if gather_rows else None

    def e2e_run(steps):
        h2d_done, comp_done, d2h_done = {}, {}, {}
        for st in range(steps):
            i = st % ROTATE
            with torch.cuda.stream(s_in):
                if st - ROTATE in comp_done:
                    s_in.wait_event(comp_done[st - ROTATE])      # a_dev[i] has been consumed
                if gather_rows:
                    a_slice[i].copy_(a_pinned_mine, non_blocking=True)
                    dist.all_gather_into_tensor(a_dev[i], a_slice[i])
                else:
                    a_dev[i].copy_(a_pinned_mine, non_blocking=True)
                h2d_done[st] = torch.cuda.Event()
                h2d_done[st].record(s_in)
            s_main.wait_event(h2d_done[st])
            if st - ROTATE in d2h_done:
                s_main.wait_event(d2h_done[st - ROTATE])         # out[i] has left the device
            quant(i)
            gemm(i)
            comp_done[st] = torch.cuda.Event()
            comp_done[st].record(s_main)
            with torch.cuda.stream(s_out):
                s_out.wait_event(comp_done[st])
                out_pinned.copy_(out[i], non_blocking=True)
                d2h_done[st] = torch.cuda.Event()
                d2h_done[st].record(s_out)
        s_main.wait_stream(s_in)
        s_main.wait_stream(s_out)

    e2e_run(3)
    barrier()
    e_start, e_stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2e_steps = max(6, min(args.steps, 20))
    e_start.record()
    e2e_run(e2e_steps)
    e_stop.record()
    barrier()
    e2e_ms = e_start.elapsed_time(e_stop)
    ks.runtime.stream_synchronize(0)

    t = torch.tensor([elapsed_ms, e2e_ms, gemm_ms, quant_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    elapsed_ms, e2e_ms, gemm_ms, quant_ms = [float(v) for v in t.tolist()]

    flops_step = 2.0 * m * N * K              # whole job, all ranks together
    flops_gemm_rank = 2.0 * m * n_local * K   # what one GEMM launch computes
    value = flops_step * args.steps / (elapsed_ms * 1e-3) / 1e12
    e2e_value = flops_step * e2e_steps / (e2e_ms * 1e-3) / 1e12
    achieved = flops_gemm_rank / (gemm_ms * 1e-3) / 1e12
    fp8_peak = 2.0 * peaks["bf16_burst"]
    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    launches_per_step = 1 + fp8_launches(m, n_local, K, sms)

    line = None
    if rank == 0:
        line = {
            "metric": "fp8_blockwise_gemm_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": elapsed_ms / args.steps,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "fp8_e4m3",
            "data": "synthetic", "config": config_of(m, world),
            "shard": {"n_per_gpu": n_local},
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": fp8_peak, "unit": "TFLOP/s",
                         "frac": achieved / fp8_peak,
                         # dram__bytes_read.sum + dram__bytes_write.sum per launch of this kernel on this
                         # workload, from one ncu capture (algorithmic bytes: 140.4e6)
                         "traffic": 149.5e6 if (world == 1 and m == M) else None,
                         "traffic_source": "one ncu capture (--set full) of fp8_blockwise_umma_kernel on this workload, "
                                           "dram__bytes_read.sum (102.9 MB) + dram__bytes_write.sum (46.7 MB) per "
                                           "launch; a constant from that capture, not a measurement of this run",
                         "kernel": "fp8_blockwise_umma_kernel", "us_per_launch": gemm_ms * 1e3,
                         "peak_source": f"2 x {peaks['source']} burst cuBLAS bf16 ({peaks['bf16_burst']} TFLOP/s): the "
                                        "timed region is milliseconds long; no FP8 figure was measured on this pool",
                         "frac_of_2x_sustained_bf16": achieved / (2.0 * peaks["bf16_sustained"]),
                         "frac_of_nominal_4500": achieved / 4500.0,
                         "quantizer_us": quant_ms * 1e3,
                         "quantizer_gbs": (m * K * 3 + m * (K // 128) * 4) / (quant_ms * 1e-3) / 1e9,
                         "quantizer_frac_of_measured_hbm": (m * K * 3 + m * (K // 128) * 4) / (quant_ms * 1e-3) / 1e9
                                                           / peaks["hbm_gbs"]},
            "e2e": {"value": e2e_value, "unit": "TFLOP/s",
                    "h2d_bytes_per_step": a_pinned_mine.numel() * 2 * world,
                    "d2h_bytes_per_step": out_pinned.numel() * 2 * world, "steps": e2e_steps,
                    "pipeline": "copy-in, kernels and copy-out of consecutive steps overlap (three streams, three "
                                "buffer sets)" + ("; every rank copies 1/N of the rows from the host and the ranks "
                                                  "all-gather them over NVLink" if gather_rows else "")},
            "gpu_launches": launches_per_step * args.steps,
            "clocks": clocks,
        }
    if not args.no_extras:
        del a_dev, b_dev, a8, out
        torch.cuda.empty_cache()
        extras = {}
        if world == 1:
            for name, fn in (("shape_7168", lambda: shape_7168(ks, torch, dev, peaks)),
                             ("w4a16_decode", lambda: w4a16_decode_sweep(ks, torch, dev, peaks)),
                             ("moe_layer", lambda: run_cfg4(args, torch, dist, ks, parallel, dev, rank, world)),
                             ("competitors", lambda: competitor_rows(ks, torch, dev))):
                try:  # secondary figures never take the headline down
                    extras[name] = fn()
                except Exception as exc:
                    extras[name] = f"failed: {type(exc).__name__}: {str(exc)[:300]}"
                torch.cuda.empty_cache()
            sec, runs, threads = cpu_step_seconds(a_cpu, b8_cpu, bs_cpu)
            extras["cpu_baseline"] = {"value": flops_step / sec / 1e12, "unit": "TFLOP/s", "cores": threads,
                                      "kind": "port", "seconds_per_step": sec,
                                      "sample": "the whole step on the host (oracle: quantizer + dequant + fp32 "
                                                f"matmul), median of {runs} runs"}
        else:
            for name, fn in (("cfg5", run_cfg5), ("cfg4", run_cfg4)):
                try:
                    extras[name] = fn(args, torch, dist, ks, parallel, dev, rank, world)
                except Exception as exc:
                    extras[name] = f"failed: {type(exc).__name__}: {str(exc)[:300]}"
                torch.cuda.empty_cache()
        if rank == 0:
            line.update(extras)
    if rank == 0:
        print(json.dumps(line), flush=True)

    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
