#!/usr/bin/env python
"""Times one kernel of the library in isolation (CUDA events, warm-up, L2 flushed between iterations) and
prints achieved throughput against the measured peaks.  Also the command line used for ncu captures:

    python scripts/kernel_bench.py gemm --m 8192 --n 6144 --k 1024
    python scripts/kernel_bench.py attn_fwd --batch 8 --seq 1024 --hq 16 --hkv 8
    python scripts/kernel_bench.py attn_bwd --batch 8 --seq 1024 --hq 16 --hkv 8
    python scripts/kernel_bench.py rmsnorm --m 8192 --h 1024
    python scripts/kernel_bench.py paged_decode --batch 256 --ctx 1024
    python scripts/kernel_bench.py sampler --batch 256
    python scripts/kernel_bench.py adamw --n 100000000
"""
import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

from b200fw import ops  # noqa: E402
from b200fw.obs.profilers import measured_peaks  # noqa: E402

DEV = "cuda"


def timeit(fn, iters, warmup, flush):
    scratch = torch.empty(256 * 1024 * 1024 // 4, device=DEV) if flush else None
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        if scratch is not None:
            scratch.zero_()          # 256 MiB write: evicts the 126 MB L2
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        times.append(s.elapsed_time(e))
    times.sort()
    return times[len(times) // 2], times[0]


def main():
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("kernel", choices=["gemm", "attn_fwd", "attn_bwd", "rmsnorm", "rmsnorm_bwd", "qknorm_rope", "swiglu",
                                       "lmhead_ce", "paged_decode", "sampler", "adamw", "kv_store"])
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=6144)
    ap.add_argument("--k", type=int, default=1024)
    ap.add_argument("--h", type=int, default=1024)
    ap.add_argument("--a-mn", type=int, default=0)
    ap.add_argument("--b-mn", type=int, default=0)
    ap.add_argument("--bn", type=int, default=0)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--seq", type=int, default=1024)
    ap.add_argument("--hq", type=int, default=16)
    ap.add_argument("--hkv", type=int, default=8)
    ap.add_argument("--ctx", type=int, default=1024)
    ap.add_argument("--vocab", type=int, default=151936)
    ap.add_argument("--fp8", action="store_true")
    ap.add_argument("--fp32-acc", action="store_true", help="gemm: accumulate into an fp32 output (weight-gradient form)")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--no-flush", action="store_true")
    a = ap.parse_args()
    torch.manual_seed(0)
    peaks = measured_peaks()
    bf = torch.bfloat16
    flops = bytes_ = 0.0
    if a.kernel == "gemm":
        A = torch.randn((a.k, a.m) if a.a_mn else (a.m, a.k), device=DEV, dtype=bf)
        B = torch.randn((a.k, a.n) if a.b_mn else (a.n, a.k), device=DEV, dtype=bf)
        C = torch.zeros(a.m, a.n, device=DEV, dtype=torch.float32 if a.fp32_acc else bf)
        fn = lambda: ops.gemm(A, B, a_mn=bool(a.a_mn), b_mn=bool(a.b_mn), out=C, bn=a.bn, accumulate=a.fp32_acc)
        flops = 2.0 * a.m * a.n * a.k
        bytes_ = 2.0 * (a.m * a.k + a.n * a.k + a.m * a.n)
    elif a.kernel in ("attn_fwd", "attn_bwd"):
        T, D = a.batch * a.seq, 128
        q = torch.randn(T, a.hq * D, device=DEV, dtype=bf, requires_grad=True)
        k = torch.randn(T, a.hkv * D, device=DEV, dtype=bf, requires_grad=True)
        v = torch.randn(T, a.hkv * D, device=DEV, dtype=bf, requires_grad=True)
        fwd_flops = 4.0 * a.batch * a.hq * a.seq * a.seq * D / 2
        if a.kernel == "attn_fwd":
            with torch.no_grad():
                fn = lambda: ops.flash_attention(q, k, v, a.batch, a.seq, a.hq, a.hkv)
                fn()
            no_grad = torch.no_grad()
            no_grad.__enter__()
            flops = fwd_flops
        else:
            o = ops.flash_attention(q, k, v, a.batch, a.seq, a.hq, a.hkv)
            g = torch.randn_like(o)
            fn = lambda: torch.autograd.grad(o, (q, k, v), g, retain_graph=True)
            flops = 2.5 * fwd_flops
        bytes_ = 2.0 * T * D * (2 * a.hq + 2 * a.hkv)
    elif a.kernel in ("rmsnorm", "rmsnorm_bwd"):
        x = torch.randn(a.m, a.h, device=DEV, dtype=bf, requires_grad=True)
        w = torch.ones(a.h, device=DEV, dtype=bf, requires_grad=True)
        if a.kernel == "rmsnorm":
            torch.set_grad_enabled(False)
            fn = lambda: ops.rmsnorm(x, w)
            bytes_ = 4.0 * a.m * a.h
        else:
            y = ops.rmsnorm(x, w)
            g = torch.randn_like(y)
            fn = lambda: torch.autograd.grad(y, (x, w), g, retain_graph=True)
            bytes_ = 6.0 * a.m * a.h
    elif a.kernel == "qknorm_rope":
        torch.set_grad_enabled(False)
        qkv = torch.randn(a.m, (a.hq + 2 * a.hkv) * 128, device=DEV, dtype=bf)
        qw = torch.ones(128, device=DEV, dtype=bf)
        pos = torch.arange(a.m, device=DEV, dtype=torch.int32) % 4096
        cos, sin = ops.rope_tables(4096, 128, 1e6, DEV)
        fn = lambda: ops.qknorm_rope(qkv, qw, qw, pos, cos, sin, a.hq, a.hkv, 128)
        bytes_ = 4.0 * a.m * (a.hq + a.hkv) * 128
    elif a.kernel == "swiglu":
        torch.set_grad_enabled(False)
        gu = torch.randn(a.m, 2 * a.n, device=DEV, dtype=bf)
        fn = lambda: ops.swiglu(gu)
        bytes_ = 6.0 * a.m * a.n
    elif a.kernel == "lmhead_ce":
        h = (0.1 * torch.randn(a.m, a.h, device=DEV)).to(bf).requires_grad_()
        w = (0.02 * torch.randn(a.vocab, a.h, device=DEV)).to(bf).requires_grad_()
        labels = torch.randint(0, a.vocab, (a.m,), device=DEV)
        def fn():
            w.grad = None
            h.grad = None
            ops.lm_head_cross_entropy(h, w, labels).backward()
        flops = 6.0 * a.m * a.h * a.vocab
    elif a.kernel == "paged_decode":
        torch.set_grad_enabled(False)
        nblk = a.batch * ((a.ctx + 15) // 16) + 1
        dt = torch.uint8 if a.fp8 else bf
        kc = torch.zeros(nblk, 16, a.hkv, 128, dtype=dt, device=DEV)
        vc = torch.zeros_like(kc)
        if not a.fp8:
            kc.normal_()
            vc.normal_()
        ks = torch.ones(nblk, a.hkv, device=DEV) if a.fp8 else None
        per = (a.ctx + 15) // 16
        bt = (torch.arange(a.batch * per, device=DEV, dtype=torch.int32).reshape(a.batch, per))
        cl = torch.full((a.batch,), a.ctx, device=DEV, dtype=torch.int32)
        q = torch.randn(a.batch, a.hq * 128, device=DEV, dtype=bf)
        need_split = a.batch * a.hkv < 296
        part = 512 if need_split else 0
        ns = (a.ctx + 511) // 512 if need_split else 1
        fn = lambda: ops.paged_decode_attention(q, kc, vc, bt, cl, a.hq, k_scale=ks, v_scale=ks, partition=part, nsplit=ns)
        bytes_ = 2.0 * a.batch * a.ctx * a.hkv * 128 * (1 if a.fp8 else 2)
    elif a.kernel == "sampler":
        torch.set_grad_enabled(False)
        logits = (3 * torch.randn(a.batch, a.vocab, device=DEV)).to(bf)
        t = torch.full((a.batch,), 0.8, device=DEV)
        p = torch.full((a.batch,), 0.95, device=DEV)
        u = torch.rand(a.batch, device=DEV)
        fn = lambda: ops.topp_sample(logits, t, p, u)
        bytes_ = 2.0 * a.batch * a.vocab
    elif a.kernel == "adamw":
        n = a.n if a.n > 1_000_000 else 100_000_000
        master = torch.randn(n, device=DEV)
        m_, v_ = torch.zeros_like(master), torch.zeros_like(master)
        g = torch.randn(n, device=DEV).to(bf)
        out = torch.empty(n, device=DEV, dtype=bf)
        hyper = torch.tensor([1e-4, 0.9, 0.999, 1e-8, 0.01, 0.1, 0.001, 1.0], device=DEV)
        fn = lambda: ops.fused_adamw(master, m_, v_, g, hyper, param_out=out)
        bytes_ = n * (12 + 12 + 2 + 2)
    elif a.kernel == "kv_store":
        torch.set_grad_enabled(False)
        nblk = a.m // 16 + 1
        dt = torch.uint8 if a.fp8 else bf
        kc = torch.zeros(nblk, 16, a.hkv, 128, dtype=dt, device=DEV)
        vc = torch.zeros_like(kc)
        ks = torch.zeros(nblk, a.hkv, device=DEV) if a.fp8 else None
        vs = torch.zeros(nblk, a.hkv, device=DEV) if a.fp8 else None
        k = torch.randn(a.m, a.hkv * 128, device=DEV, dtype=bf)
        segs = torch.tensor([[i, 16 * i, 16, 0] for i in range(a.m // 16)], dtype=torch.int32, device=DEV)
        fn = lambda: ops.kv_store(k, k, kc, vc, segs, ks, vs)
        bytes_ = a.m * a.hkv * 128 * 2 * (2 + (1 if a.fp8 else 2))
    med, best = timeit(fn, a.iters, a.warmup, not a.no_flush)
    out = {"kernel": a.kernel, "ms_median": med, "ms_best": best, "peaks": peaks["source"]}
    if flops:
        out["tflops"] = flops / (med * 1e-3) / 1e12
        out["frac_of_measured_bf16_burst"] = out["tflops"] / peaks["bf16_tflops"]
    if bytes_:
        out["gbs"] = bytes_ / (med * 1e-3) / 1e9
        out["frac_of_measured_hbm"] = out["gbs"] / peaks["hbm_gbs"]
    print(json.dumps(out))


if __name__ == "__main__":
    main()
