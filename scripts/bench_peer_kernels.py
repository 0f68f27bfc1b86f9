#!/usr/bin/env python
"""Peer-memory kernels against their roofline: the ZeRO gradient reduce (every rank sums its shard out of
all peers' gradient buckets), the ZeRO AdamW + publish (update the shard, write the bf16 result into every
peer's parameter bucket) and the weight-sync peer write (cast + checksum into a receiver's staging buffer).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 scripts/bench_peer_kernels.py

Device-timed with CUDA events on the launching stream, max over ranks, 3 warm-ups.  Roofline: bytes that
must cross NVLink divided by the measured peer-copy bandwidth (770 GB/s per direction per GPU), or local HBM
bytes over the measured copy bandwidth, whichever is slower.
"""
import argparse
import ctypes
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

from b200fw import _native as nv  # noqa: E402
from b200fw.dist.symm import FlagBarrier, SymmetricBuffer  # noqa: E402
from b200fw.obs.profilers import measured_peaks  # noqa: E402

LINK_GBS = 770.0


def timed(fn, barrier, iters, warmup):
    for _ in range(warmup):
        barrier()
        fn()
    ts = []
    for _ in range(iters):
        barrier()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        ts.append(s.elapsed_time(e))
    ts.sort()
    t = torch.tensor([ts[len(ts) // 2]], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def main():
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--params", type=int, default=600_000_000, help="parameters in the bucket set (Qwen3-0.6B: 0.6e9)")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    a = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    nv.set_device(local)
    group = dist.group.WORLD
    peaks = measured_peaks()
    hbm = peaks["hbm_gbs"]
    n = (a.params // (world * 1024)) * world * 1024
    shard = n // world
    L = nv.lib()
    grads = SymmetricBuffer(n, torch.bfloat16, group)         # bf16 gradient bucket of the peer-memory ZeRO path
    params = SymmetricBuffer(n, torch.bfloat16, group)        # bf16 parameter bucket
    grads.tensor.normal_(0, 1e-3)
    flags = FlagBarrier(group)
    barrier = lambda: flags.barrier(1)
    out = torch.empty(shard, device="cuda")
    norm = torch.zeros(1, device="cuda")
    master = torch.zeros(shard, device="cuda")
    m = torch.zeros(shard, device="cuda")
    v = torch.zeros(shard, device="cuda")
    hyper = torch.tensor([1e-5, 0.9, 0.999, 1e-8, 0.01, 0.1, 0.001, 1.0], device="cuda")
    res = []
    from b200fw.obs.clocks import ClockSampler
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()

    def reduce():
        nv.check(L.b2_zero_reduce_shard(grads.ptr_array, world, ctypes.c_longlong(rank * shard), ctypes.c_longlong(shard),
                                        ctypes.c_float(1.0 / world), nv.ptr(out), 0, nv.ptr(norm), nv.stream_ptr()),
                 "zero_reduce_shard")

    t = timed(reduce, barrier, a.iters, a.warmup)
    wire = shard * 2 * (world - 1)                              # this rank pulls its bf16 shard from every peer
    local_bytes = shard * (2 + 4)                               # own slice read + fp32 result written
    roof = max(wire / (LINK_GBS * 1e9), local_bytes / (hbm * 1e9)) * 1e3
    res.append({"kernel": "zero_reduce_shard", "ms": t, "wire_mb": wire / 1e6, "roofline_ms": roof,
                "roofline_fraction": roof / t, "pull_gbs": wire / t / 1e6})

    def publish():
        nv.check(L.b2_zero_adamw_publish(nv.ptr(master), nv.ptr(m), nv.ptr(v), nv.ptr(out), ctypes.c_longlong(shard),
                                         nv.ptr(hyper), nv.ptr(norm), params.ptr_array, world,
                                         ctypes.c_longlong(rank * shard), nv.stream_ptr()), "zero_adamw_publish")

    if grads.mc_ptr:
        def reduce_mc():
            nv.check(L.b2_zero_reduce_shard_mc(ctypes.c_void_p(grads.mc_ptr), ctypes.c_longlong(rank * shard),
                                               ctypes.c_longlong(shard), ctypes.c_float(1.0 / world), nv.ptr(out), 0,
                                               nv.ptr(norm), nv.stream_ptr()), "zero_reduce_shard_mc")
        t = timed(reduce_mc, barrier, a.iters, a.warmup)
        res.append({"kernel": "zero_reduce_shard (multimem.ld_reduce through the switch)", "ms": t, "wire_mb": wire / 1e6,
                    "roofline_ms": roof, "roofline_fraction": roof / t, "served_gbs": wire / t / 1e6})
    # the library form of the same step: NCCL reduce-scatter of the bf16 bucket
    rs_out = torch.empty(shard, device="cuda", dtype=torch.bfloat16)
    t = timed(lambda: dist.reduce_scatter_tensor(rs_out, grads.tensor), barrier, a.iters, a.warmup)
    res.append({"kernel": "NCCL reduce_scatter (bf16, same bucket)", "ms": t, "wire_mb": wire / 1e6, "roofline_ms": roof,
                "roofline_fraction": roof / t})

    norm.fill_(1.0)
    t = timed(publish, barrier, a.iters, a.warmup)
    wire = shard * 2 * (world - 1)                              # bf16 result pushed to every peer
    local_bytes = shard * (4 * 7 + 2)                           # master, m, v read + written, grad read, own bf16 copy
    roof = max(wire / (LINK_GBS * 1e9), local_bytes / (hbm * 1e9)) * 1e3
    res.append({"kernel": "zero_adamw_publish", "ms": t, "wire_mb": wire / 1e6, "hbm_mb": local_bytes / 1e6,
                "roofline_ms": roof, "roofline_fraction": roof / t})

    if params.mc_ptr:
        ok = torch.ones(1, dtype=torch.int32, device="cuda")

        def publish_mc():
            nv.check(L.b2_zero_adamw_publish2(nv.ptr(master), nv.ptr(m), nv.ptr(v), nv.ptr(out), ctypes.c_longlong(shard),
                                              nv.ptr(hyper), nv.ptr(norm), params.ptr_array, ctypes.c_void_p(params.mc_ptr),
                                              world, ctypes.c_longlong(rank * shard), nv.ptr(ok), nv.stream_ptr()),
                     "zero_adamw_publish2")
        t = timed(publish_mc, barrier, a.iters, a.warmup)
        res.append({"kernel": "zero_adamw_publish (multimem.st through the switch)", "ms": t, "wire_mb": wire / 1e6,
                    "hbm_mb": local_bytes / 1e6, "roofline_ms": roof, "roofline_fraction": roof / t})
    t = timed(lambda: dist.all_gather_into_tensor(params.tensor, params.tensor[rank * shard:(rank + 1) * shard]), barrier,
              a.iters, a.warmup)
    res.append({"kernel": "NCCL all_gather (bf16, same bucket; AdamW not included)", "ms": t, "wire_mb": wire / 1e6})

    # weight sync: rank 0's fp32 master shard -> bf16 staging buffer on the next rank (cast + checksum)
    src = torch.randn(n // 2, device="cuda")
    stage = SymmetricBuffer(n // 2, torch.bfloat16, group)
    csum = torch.zeros(2, dtype=torch.int64, device="cuda")
    dst_ptr = ctypes.c_void_p(stage.peer_ptrs[(rank + 1) % world])

    def push():
        nv.check(L.b2_peer_write(nv.ptr(src), 1, dst_ptr, 0, ctypes.c_longlong(n // 2), ctypes.c_longlong(0), 0,
                                 nv.ptr(csum), nv.stream_ptr()), "peer_write")

    t = timed(push, barrier, a.iters, a.warmup)
    wire = (n // 2) * 2
    roof = max(wire / (LINK_GBS * 1e9), (n // 2) * 4 / (hbm * 1e9)) * 1e3
    res.append({"kernel": "peer_write fp32->bf16 + checksum", "ms": t, "wire_mb": wire / 1e6, "roofline_ms": roof,
                "roofline_fraction": roof / t, "push_gbs": wire / t / 1e6})
    # ---- the whole weight sync through the public class: Qwen3-0.6B state dict (310 tensors, 1.19 GB bf16) from
    # rank 0 into every other rank's staging image, checksum verified there, version committed.  Timed like the
    # reference arm (baseline/run_reference_extras.py sync): host clock around a device sync, max over ranks.
    import time
    from b200fw.model.config import PRESETS
    from b200fw.sync import PeerWeightSync
    mc = PRESETS["qwen3-0.6b"]
    H, D, I = mc.hidden_size, mc.head_dim, mc.intermediate_size
    layout = [("model.embed_tokens.weight", (mc.vocab_size, H)), ("model.norm.weight", (H,))]
    for i in range(mc.num_layers):
        p = f"model.layers.{i}."
        layout += [(p + "self_attn.q_proj.weight", (mc.num_heads * D, H)), (p + "self_attn.k_proj.weight", (mc.num_kv_heads * D, H)),
                   (p + "self_attn.v_proj.weight", (mc.num_kv_heads * D, H)), (p + "self_attn.o_proj.weight", (H, mc.num_heads * D)),
                   (p + "self_attn.q_norm.weight", (D,)), (p + "self_attn.k_norm.weight", (D,)),
                   (p + "mlp.gate_proj.weight", (I, H)), (p + "mlp.up_proj.weight", (I, H)), (p + "mlp.down_proj.weight", (H, I)),
                   (p + "input_layernorm.weight", (H,)), (p + "post_attention_layernorm.weight", (H,))]
    ps = PeerWeightSync(layout, torch.bfloat16, group=group, sender_rank=0)
    state = {k: torch.full(shape, 0.01, dtype=torch.bfloat16, device="cuda") for k, shape in layout} if rank == 0 else None

    class _Sink:
        def load_weights(self, views):
            pass

    sync_ms = []
    for it in range(a.warmup + 5):
        dist.barrier()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        ps.sync(rank == 0, state, None if rank == 0 else _Sink())
        torch.cuda.synchronize()
        dt = torch.tensor([time.perf_counter() - t0], dtype=torch.float64, device="cuda")
        dist.all_reduce(dt, op=dist.ReduceOp.MAX)
        if it >= a.warmup:
            sync_ms.append(float(dt) * 1e3)
    sync_ms.sort()
    nbytes = sum(2 * torch.Size(s_).numel() for _, s_ in layout)
    res.append({"kernel": "PeerWeightSync.sync, Qwen3-0.6B full image to every other rank (write + verify + commit + control messages)",
                "ms": sync_ms[len(sync_ms) // 2], "best_ms": sync_ms[0], "bytes_per_receiver": nbytes,
                "receivers": world - 1, "version": ps.version})
    torch.cuda.synchronize()
    status = nv.read_status()
    clocks = sampler.stop() if rank == 0 else None
    if rank == 0:
        print(json.dumps({"world": world, "params": n, "results": res, "device_status": status, "clocks": clocks,
                          "nvls_multicast": bool(grads.mc_ptr),
                          "link_gbs_measured": LINK_GBS, "hbm_gbs": hbm}, indent=1))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
