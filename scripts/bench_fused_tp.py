#!/usr/bin/env python
"""Roofline benchmark of the fused tensor-parallel GEMMs against the unfused NCCL sequence.

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 scripts/bench_fused_tp.py

Shapes: Qwen3-32B architecture at TP8 with sequence parallelism, M = 16384 tokens (per-rank weight shards:
QKV N=1280, gate|up N=6400 from K=5120; o_proj K=1024, down_proj K=3200 to N=5120).  With fewer ranks the
per-rank weight shapes stay the same and the token shard grows.  For every path it prints the device time
(CUDA events, max over ranks), the unfused time (NCCL collective + the same GEMM kernel), and the
fraction of the roofline max(FLOPs / measured bf16 peak, NVLink bytes / 770 GB/s).
"""
import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

from b200fw import _native as nv  # noqa: E402
from b200fw.obs.clocks import ClockSampler  # noqa: E402
from b200fw.obs.profilers import CommProfiler, measured_peaks  # noqa: E402
from b200fw.ops import fused_tp, gemm  # noqa: E402


def timed(fn, iters, warmup, world, dev):
    for _ in range(warmup):
        fn()
    dist.barrier()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    torch.cuda.synchronize()
    t = torch.tensor([s.elapsed_time(e) / iters], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def main():
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--tokens", type=int, default=16384)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    a = ap.parse_args()
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    nv.set_device(local)
    g = dist.group.WORLD
    peaks = measured_peaks()
    M = a.tokens
    rows = M // world
    torch.manual_seed(rank)
    out = []
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    cases = [("F1 all-gather->GEMM qkv", "ag", 1280, 5120), ("F2 all-gather->GEMM gate|up", "ag", 6400, 5120),
             ("F3 GEMM->reduce-scatter o_proj", "rs", 5120, 1024), ("F4 GEMM->reduce-scatter down_proj", "rs", 5120, 3200)]
    for name, kind, N, K in cases:
        w = torch.randn(N, K, device=dev, dtype=torch.bfloat16) * 0.05
        flops = 2.0 * M * N * K
        if kind == "ag":
            xs = torch.randn(rows, K, device=dev, dtype=torch.bfloat16)
            full = torch.empty(M, K, device=dev, dtype=torch.bfloat16)
            fused = lambda: fused_tp.allgather_gemm(xs, w, g, slot="bench")
            def unfused():
                dist.all_gather_into_tensor(full, xs)
                return gemm(full, w)
            wire = (world - 1) / world * M * K * 2
        else:
            x = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
            res = torch.randn(rows, N, device=dev, dtype=torch.bfloat16)
            o = torch.empty(rows, N, device=dev, dtype=torch.bfloat16)
            fused = lambda: fused_tp.gemm_reduce_scatter(x, w, g, residual=res)
            def unfused():
                y = gemm(x, w)
                dist.reduce_scatter_tensor(o, y)
                return o + res
            wire = (world - 1) / world * M * N * 2
        # numerics on every rank before timing: the fused kernel against NCCL + the same GEMM
        yf = fused()
        yf = (yf[0] if isinstance(yf, tuple) else yf).float()
        yu = unfused().float()
        err = ((yf - yu).abs().max() / yu.abs().max().clamp_min(1e-6)).reshape(1)
        dist.all_reduce(err, op=dist.ReduceOp.MAX)
        rel_err = float(err)
        assert rel_err < 2e-2, f"{name}: fused result differs from NCCL + GEMM on some rank (max relative error {rel_err})"
        t_f = timed(fused, a.iters, a.warmup, world, dev)
        t_u = timed(unfused, a.iters, a.warmup, world, dev)
        roof = CommProfiler.fused_roofline(flops, wire, t_f, peaks["bf16_tflops_sustained"])
        t_wire_900 = wire / 900e9 * 1e3
        out.append({"path": name, "M": M, "N": N, "K": K, "world": world, "fused_ms": t_f, "nccl_plus_gemm_ms": t_u,
                    "speedup_vs_unfused": t_u / t_f, "t_compute_ms": roof["t_compute_ms"], "t_wire_ms": roof["t_wire_ms"],
                    "bound": roof["bound"], "roofline_fraction_of_measured": roof["fraction"],
                    "roofline_fraction_at_900GBs_wire": max(roof["t_compute_ms"], t_wire_900) / t_f,
                    "max_rel_err_vs_unfused_all_ranks": rel_err})
    status = nv.read_status()
    clocks = sampler.stop() if rank == 0 else None
    if rank == 0:
        print(json.dumps({"fused_tp": out, "device_status": status, "peaks": peaks["source"], "clocks": clocks}, indent=1))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
