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
    python scripts/kernel_bench.py gemm --m 8192 --n 6144 --k 1024 --lib      # cuBLAS (torch.matmul) on the same shape
    python scripts/kernel_bench.py attn_fwd --lib                             # flash-attn 2 on the same shape
    python scripts/kernel_bench.py suite                                      # the training step's shapes, both arms

Every line carries the SM clock sampled while the kernel ran (median MHz, throttle reasons) and
``ms_x_mhz`` (milliseconds x median MHz: proportional to cycles, comparable across differently clocked boxes).
"""
import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

from b200fw import ops  # noqa: E402
from b200fw.obs.clocks import ClockSampler  # noqa: E402
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


def timed_line(name, fn, flops, bytes_, iters, warmup, flush, peaks, extra=None):
    """Time ``fn`` with the clock sampler running; one result dict."""
    sampler = ClockSampler(torch.cuda.current_device())
    sampler.start()
    # keep the GPU busy long enough for a few 200 ms clock samples
    med, best = timeit(fn, iters, warmup, flush)
    reps = 0
    import time as _t
    t0 = _t.time()
    while _t.time() - t0 < 0.7:
        fn()
        reps += 1
        if reps % 16 == 0:
            torch.cuda.synchronize()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    out = {"kernel": name, "ms_median": med, "ms_best": best, "peaks": peaks["source"], "clocks": clocks}
    if clocks.get("sm_mhz"):
        out["ms_x_mhz"] = med * clocks["sm_mhz"]
    if flops:
        out["tflops"] = flops / (med * 1e-3) / 1e12
        out["frac_of_measured_bf16_burst"] = out["tflops"] / peaks["bf16_tflops"]
    if bytes_:
        out["gbs"] = bytes_ / (med * 1e-3) / 1e9
        out["frac_of_measured_hbm"] = out["gbs"] / peaks["hbm_gbs"]
    if extra:
        out.update(extra)
    return out


def suite(a, peaks):
    """The Qwen3-0.6B training step's GEMMs (forward, input-gradient and weight-gradient forms at 8192 tokens, and
    the 16384-token forms of the 32B TP8 step) and its attention shapes, this library against cuBLAS
    (``torch.matmul``) and flash-attn 2 on the same tensors.  One JSON line per (kernel, arm)."""
    bf = torch.bfloat16
    lines = []
    gemms = [  # name, M, N, K, a_mn, b_mn, fp32 accumulate
        ("fwd qkv 8192x4096x1024", 8192, 4096, 1024, 0, 0, False),
        ("fwd gate_up 8192x6144x1024", 8192, 6144, 1024, 0, 0, False),
        ("fwd down 8192x1024x3072", 8192, 1024, 3072, 0, 0, False),
        ("dX gate_up 8192x1024x6144 (B mn-major)", 8192, 1024, 6144, 0, 1, False),
        ("dW gate_up 6144x1024x8192 (A,B mn-major, fp32 acc)", 6144, 1024, 8192, 1, 1, True),
        ("dW down 1024x3072x8192 (A,B mn-major, fp32 acc)", 1024, 3072, 8192, 1, 1, True),
        ("fwd 32b gate_up/8 16384x6400x5120", 16384, 6400, 5120, 0, 0, False),
        ("dW 32b gate_up/8 6400x5120x16384", 6400, 5120, 16384, 1, 1, True),
        ("square 8192^3", 8192, 8192, 8192, 0, 0, False),
    ]
    for name, M, N, K, amn, bmn, acc in gemms:
        A = torch.randn((K, M) if amn else (M, K), device=DEV, dtype=bf)
        B = torch.randn((K, N) if bmn else (N, K), device=DEV, dtype=bf)
        C = torch.zeros(M, N, device=DEV, dtype=torch.float32 if acc else bf)
        fl = 2.0 * M * N * K
        ours = lambda: ops.gemm(A, B, a_mn=bool(amn), b_mn=bool(bmn), out=C, accumulate=acc)
        Ab = A.t() if amn else A
        Bb = B if bmn else B.t()
        Cb = torch.zeros(M, N, device=DEV, dtype=bf)
        if acc:   # the library form of an fp32-accumulated weight gradient: bf16 GEMM, then add into fp32
            lib = lambda: C.add_(torch.matmul(Ab, Bb))
        else:
            lib = lambda: torch.matmul(Ab, Bb, out=Cb)
        lines.append(timed_line("gemm " + name, ours, fl, 0, a.iters, a.warmup, True, peaks, {"arm": "b200fw"}))
        lines.append(timed_line("gemm " + name, lib, fl, 0, a.iters, a.warmup, True, peaks, {"arm": "cublas"}))
        print(json.dumps(lines[-2]), flush=True)
        print(json.dumps(lines[-1]), flush=True)
        del A, B, C, Cb
    try:
        from flash_attn import flash_attn_func
    except Exception as e:  # noqa: BLE001
        flash_attn_func = None
        print(json.dumps({"kernel": "attention", "arm": "flash_attn", "unavailable": f"{type(e).__name__}: {e}"}))
    for batch, seq, hq, hkv in [(8, 1024, 16, 8), (8, 2048, 8, 1), (2, 8192, 16, 8)]:
        T, D = batch * seq, 128
        q = torch.randn(T, hq * D, device=DEV, dtype=bf, requires_grad=True)
        k = torch.randn(T, hkv * D, device=DEV, dtype=bf, requires_grad=True)
        v = torch.randn(T, hkv * D, device=DEV, dtype=bf, requires_grad=True)
        ff = 4.0 * batch * hq * seq * seq * D / 2
        tag = f"b{batch} s{seq} h{hq}:{hkv}"
        o = ops.flash_attention(q, k, v, batch, seq, hq, hkv)
        g = torch.randn_like(o)

        def ours_f():
            with torch.no_grad():
                ops.flash_attention(q, k, v, batch, seq, hq, hkv)
        ours_b = lambda: torch.autograd.grad(o, (q, k, v), g, retain_graph=True)
        r = [timed_line("attn_fwd " + tag, ours_f, ff, 0, a.iters, a.warmup, True, peaks, {"arm": "b200fw"}),
             timed_line("attn_bwd " + tag, ours_b, 2.5 * ff, 0, a.iters, a.warmup, True, peaks, {"arm": "b200fw"})]
        if flash_attn_func is not None:
            q4 = q.detach().view(batch, seq, hq, D).requires_grad_()
            k4 = k.detach().view(batch, seq, hkv, D).requires_grad_()
            v4 = v.detach().view(batch, seq, hkv, D).requires_grad_()
            o4 = flash_attn_func(q4, k4, v4, causal=True)
            g4 = torch.randn_like(o4)

            def lib_f():
                with torch.no_grad():
                    flash_attn_func(q4, k4, v4, causal=True)
            lib_b = lambda: torch.autograd.grad(o4, (q4, k4, v4), g4, retain_graph=True)
            r.append(timed_line("attn_fwd " + tag, lib_f, ff, 0, a.iters, a.warmup, True, peaks, {"arm": "flash_attn"}))
            r.append(timed_line("attn_bwd " + tag, lib_b, 2.5 * ff, 0, a.iters, a.warmup, True, peaks, {"arm": "flash_attn"}))
        for x in r:
            print(json.dumps(x), flush=True)
        lines += r
    return lines


def main():
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("kernel", choices=["suite", "gemm", "attn_fwd", "attn_bwd", "rmsnorm", "rmsnorm_bwd", "qknorm_rope", "swiglu",
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
    ap.add_argument("--partition", type=int, default=0, help="paged_decode: tokens per split-KV partition (0 = automatic)")
    ap.add_argument("--decode-mode", default=None, choices=["0", "3"],
                    help="paged_decode: row loop of the kernel (0 registers, 3 cp.async ring)")
    ap.add_argument("--fp32-acc", action="store_true", help="gemm: accumulate into an fp32 output (weight-gradient form)")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--no-flush", action="store_true")
    ap.add_argument("--lib", action="store_true",
                    help="time the library counterpart instead (gemm: torch.matmul / cuBLAS; attn_*: flash-attn 2)")
    a = ap.parse_args()
    torch.manual_seed(0)
    peaks = measured_peaks()
    bf = torch.bfloat16
    flops = bytes_ = 0.0
    if a.kernel == "suite":
        suite(a, peaks)
        return
    if a.kernel == "gemm":
        A = torch.randn((a.k, a.m) if a.a_mn else (a.m, a.k), device=DEV, dtype=bf)
        B = torch.randn((a.k, a.n) if a.b_mn else (a.n, a.k), device=DEV, dtype=bf)
        C = torch.zeros(a.m, a.n, device=DEV, dtype=torch.float32 if a.fp32_acc else bf)
        fn = lambda: ops.gemm(A, B, a_mn=bool(a.a_mn), b_mn=bool(a.b_mn), out=C, bn=a.bn, accumulate=a.fp32_acc)
        if a.lib:
            Ab, Bb = (A.t() if a.a_mn else A), (B if a.b_mn else B.t())
            Cb = torch.zeros(a.m, a.n, device=DEV, dtype=bf)
            fn = (lambda: C.add_(torch.matmul(Ab, Bb))) if a.fp32_acc else (lambda: torch.matmul(Ab, Bb, out=Cb))
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
        if a.lib:
            from flash_attn import flash_attn_func
            q4 = q.detach().view(a.batch, a.seq, a.hq, D).requires_grad_()
            k4 = k.detach().view(a.batch, a.seq, a.hkv, D).requires_grad_()
            v4 = v.detach().view(a.batch, a.seq, a.hkv, D).requires_grad_()
            if a.kernel == "attn_fwd":
                fn = lambda: flash_attn_func(q4, k4, v4, causal=True)
            else:
                torch.set_grad_enabled(True)
                o4 = flash_attn_func(q4, k4, v4, causal=True)
                g4 = torch.randn_like(o4)
                fn = lambda: torch.autograd.grad(o4, (q4, k4, v4), g4, retain_graph=True)
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
        if a.decode_mode is not None:
            os.environ["B200FW_DECODE_MODE"] = a.decode_mode
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
        if a.partition:
            part, ns = a.partition, (a.ctx + a.partition - 1) // a.partition
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
    out = timed_line(a.kernel, fn, flops, bytes_, a.iters, a.warmup, not a.no_flush, peaks,
                     {"arm": "library" if a.lib else "b200fw"})
    print(json.dumps(out))


if __name__ == "__main__":
    main()
