"""Headline benchmark: full-SFT training throughput (tokens/s) and MFU.

Default workload (one named by the benchmark configs): Qwen3-0.6B-architecture full SFT in bf16, data
parallel over N GPUs with ZeRO-1, sequence 1024, micro-batch 8 per GPU, gradient accumulation 2,
seeded uniform synthetic tokens with the loss on the second half of every sequence, random-init
weights.  ``--model qwen3-32b --tp 8`` runs the TP8 large-model configuration on 8 GPUs.

One "step" is one optimizer step (all its micro-batches, gradient reduction, clip, AdamW).  Prints one
JSON line on rank 0.  ``--impl reference`` runs the unmodified reference implementation installed under
``baseline/_ref`` on the same workload through its own TrainEngine.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from b200fw.obs.clocks import ClockSampler  # noqa: E402


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200fw", choices=["b200fw", "reference"])
    ap.add_argument("--model", default="qwen3-0.6b")
    ap.add_argument("--seq-len", type=int, default=1024)
    ap.add_argument("--micro-batch", type=int, default=8)
    ap.add_argument("--grad-accum", type=int, default=2)
    ap.add_argument("--zero-stage", type=int, default=1)
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--pp", type=int, default=1)
    ap.add_argument("--lora-rank", type=int, default=0)
    ap.add_argument("--grad-ckpt", action="store_true")
    ap.add_argument("--sequence-parallel", action="store_true")
    ap.add_argument("--zero-comm", default="auto", choices=["auto", "nccl", "p2p"],
                    help="ZeRO gradient reduce-scatter / parameter all-gather: inside the optimizer kernels over peer memory "
                         "(p2p), NCCL, or auto (p2p for plain data parallelism with ZeRO-1, NCCL otherwise)")
    ap.add_argument("--no-zero3-prefetch", dest="zero3_prefetch", action="store_false",
                    help="ZeRO-3: wait for every parameter gather before the forward instead of layer by layer")
    ap.add_argument("--no-cuda-graph", dest="cuda_graph", action="store_false",
                    help="launch the micro-step kernel by kernel instead of replaying forward + backward as one CUDA "
                         "graph (the graph path applies to DP / single GPU with ZeRO <= 1; other layouts run eagerly)")
    ap.add_argument("--graph-reduce", dest="graph_reduce", action="store_true", default=None,
                    help="capture the gradient reduce-scatters inside the last micro-batch's CUDA graph, overlapped with "
                         "its backward (default: on for the p2p ZeRO backend, off for NCCL)")
    ap.add_argument("--no-graph-reduce", dest="graph_reduce", action="store_false")
    ap.add_argument("--layers", type=int, default=0,
                    help="override the preset's layer count (smoke runs of a large architecture; not a benchmark config)")
    ap.add_argument("--fused-tp", action="store_true",
                    help="run the sequence-parallel collectives inside the GEMM kernels (peer memory) instead of NCCL")
    return ap.parse_args()


def synthetic_batches(vocab, micro_batch, seq, count, seed, pinned):
    g = torch.Generator().manual_seed(seed)
    out = []
    for _ in range(count):
        ids = torch.randint(0, vocab, (micro_batch, seq), generator=g, dtype=torch.long)
        labels = ids.clone()
        labels[:, : seq // 2] = -100
        if pinned:
            ids, labels = ids.pin_memory(), labels.pin_memory()
        out.append((ids, labels))
    return out


def max_over_ranks(x: float, world: int, device) -> float:
    if world == 1:
        return x
    import torch.distributed as dist
    t = torch.tensor([x], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def run_ours(a):
    from b200fw import _native as nv
    from b200fw.model import PRESETS
    from b200fw.obs.profilers import ComputeProfiler, measured_peaks
    from b200fw.train import TrainConfig, TrainEngine

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    assert world == a.gpus, f"--gpus {a.gpus} but WORLD_SIZE={world}"
    torch.cuda.set_device(local)
    dp = world // (a.tp * a.pp)
    import copy
    mc = copy.deepcopy(PRESETS[a.model])
    if a.layers > 0:
        mc.num_layers = a.layers
    cfg = TrainConfig(model_config=mc, tp_size=a.tp, dp_size=dp, pp_size=a.pp,
                      num_micro_batches=max(a.pp, a.grad_accum) if a.pp > 1 else 1, max_seq_len=a.seq_len,
                      use_gradient_checkpoint=a.grad_ckpt, lora_rank=a.lora_rank, learning_rate=1e-5,
                      gradient_accumulation_steps=a.grad_accum if a.pp == 1 else 1, grpo_beta=0.0,
                      zero_stage=a.zero_stage, warmup_steps=2, total_training_steps=a.steps + a.warmup + 8,
                      sequence_parallel=a.sequence_parallel, amp_dtype="bf16", zero_comm_backend=a.zero_comm,
                      fused_tp_comm=a.fused_tp, cuda_graph_step=a.cuda_graph, zero3_prefetch=a.zero3_prefetch,
                      cuda_graph_reduce=a.graph_reduce)
    eng = TrainEngine(cfg).initialize()
    dev = eng.device
    accum = a.grad_accum
    n_micro = (a.warmup + a.steps) * accum
    host = synthetic_batches(mc.vocab_size, a.micro_batch, a.seq_len, accum * 2, 1234 + eng.parallel_ctx.dp_rank, True)
    on_dev = [(i.to(dev), l.to(dev)) for i, l in host]
    # the same batches as the token lists the public step takes (prompt = unsupervised half, response = the rest)
    half = a.seq_len // 2
    as_lists = [([r[:half].tolist() for r in i], [r[half:].tolist() for r in i]) for i, _ in host]

    def micro_dev(k):
        ids, labels = on_dev[k % len(on_dev)]
        if a.pp > 1:
            return eng.sft_step_tensors(ids, labels, sync=False)
        return eng.sft_step_tensors(ids, labels, sync=False)

    def barrier():
        if world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize()

    micro_per_step = accum if a.pp == 1 else 1
    # ---- device-timed: inputs resident on the device, no host sync inside the region ----------------
    for k in range(a.warmup * micro_per_step):
        micro_dev(k)
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    launches0 = nv.launch_count
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for k in range(a.steps * micro_per_step):
        micro_dev(k)
    e.record()
    barrier()
    ms = max_over_ranks(s.elapsed_time(e), world, dev)
    launches = nv.launch_count - launches0
    status = nv.read_status()
    # ---- end to end through the public step: TrainEngine.sft_step(prompt token lists, response token lists),
    # the call the orchestrators make.  Inside it, every micro-batch: lists -> pinned host buffer -> device copy
    # (ids, labels, supervised-row indices), and the loss (and the gradient norm on optimizer steps) read back.
    barrier()
    s2, e2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s2.record()
    last_loss, h2d = 0.0, 0
    for k in range(a.steps * micro_per_step):
        if a.pp > 1:
            ids, labels = host[k % len(host)]
            m = eng.sft_step_tensors(ids, labels, sync=True)
        else:
            m = eng.sft_step(*as_lists[k % len(as_lists)])
        h2d += eng.last_h2d_bytes
        last_loss = m.loss
    e2.record()
    barrier()
    ms_e2e = max_over_ranks(s2.elapsed_time(e2), world, dev)
    clocks = sampler.stop() if rank == 0 else None

    tokens_per_step = a.micro_batch * a.seq_len * micro_per_step * dp * (a.grad_accum if a.pp > 1 and False else 1)
    tps = tokens_per_step * a.steps / (ms * 1e-3)
    tps_e2e = tokens_per_step * a.steps / (ms_e2e * 1e-3)
    # executed FLOPs: the LM head runs on the supervised rows only (half of every sequence here); the forward
    # that gradient checkpointing repeats counts for hardware utilisation (HFU), not for model FLOPs (MFU)
    sup = (a.seq_len - a.seq_len // 2) / a.seq_len
    gb = a.micro_batch * micro_per_step * dp
    flops = ComputeProfiler.exact_flops(mc, gb, a.seq_len, full=a.lora_rank <= 0, grad_checkpoint=a.grad_ckpt,
                                        supervised_fraction=sup)
    flops_hw = ComputeProfiler.exact_flops(mc, gb, a.seq_len, full=a.lora_rank <= 0, grad_checkpoint=a.grad_ckpt,
                                           supervised_fraction=sup, count_recompute=True)
    peaks = measured_peaks()
    step_s = ms * 1e-3 / a.steps
    if rank == 0:
        par = "+".join(p for p in [f"dp{dp}" if dp > 1 or (a.tp == 1 and a.pp == 1) else "", f"tp{a.tp}" if a.tp > 1 else "",
                                   f"pp{a.pp}" if a.pp > 1 else ""] if p)
        line = {
            "metric": "sft_tokens_per_s", "value": tps, "unit": "tokens/s", "n_gpus": world, "steps": a.steps,
            "warmup": a.warmup, "ms_per_step": ms / a.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic (seeded uniform tokens, random-init weights)",
            "impl": "b200fw",
            "config": {"model": (f"{a.model}-arch full SFT" if a.lora_rank <= 0 else f"{a.model}-arch LoRA r{a.lora_rank}")
                       + (f" (layers cut to {a.layers}: smoke run, not the named config)" if a.layers > 0 else ""),
                       "global_batch": a.micro_batch * micro_per_step * dp, "micro_batch_per_gpu": a.micro_batch,
                       "grad_accum": a.grad_accum, "seq_len": a.seq_len, "parallelism": par,
                       "zero_stage": a.zero_stage, "zero_comm": getattr(eng.optimizer, "comm_backend", a.zero_comm) if world > 1 else "none (1 GPU)",
                       "zero_nvls": bool(getattr(eng.optimizer, "nvls", False)), "zero3_prefetch": a.zero3_prefetch,
                       "sequence_parallel": a.sequence_parallel, "fused_tp_comm": a.fused_tp, "grad_ckpt": a.grad_ckpt,
                       "cuda_graph_step": a.cuda_graph, "cuda_graph_reduce": a.graph_reduce, "l2": "inputs larger than L2 (weights+activations >> 126 MB)",
                       "step": "one optimizer step = grad_accum micro-batches + reduce + clip + AdamW"},
            "mfu_model_of_measured_sustained": flops / (step_s * world * peaks["bf16_tflops_sustained"] * 1e12),
            "hfu_of_measured_sustained": flops_hw / (step_s * world * peaks["bf16_tflops_sustained"] * 1e12),
            "model_tflops_per_gpu": flops / step_s / world / 1e12,
            "flops_note": "LM head counted on the supervised rows only; hfu adds the checkpoint recompute",
            "e2e": {"value": tps_e2e, "unit": "tokens/s", "ms_per_step": ms_e2e / a.steps,
                    "h2d_bytes_per_step": h2d // a.steps,
                    "d2h_bytes_per_step": 4 * micro_per_step + 8, "final_loss": last_loss,
                    "api": "TrainEngine.sft_step(prompt token lists, response token lists)" if a.pp == 1
                           else "TrainEngine.sft_step_tensors(pinned host tensors)"},
            "gpu_launches": launches, "device_status": status, "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    # the result is out; a teardown that hangs or raises still fails the run (exit code 3 / the exception)
    def _hung():
        print("[bench] teardown did not finish within 120 s", file=sys.stderr, flush=True)
        os._exit(3)
    guard = threading.Timer(120.0, _hung)
    guard.daemon = True
    guard.start()
    eng.parallel_ctx.destroy()
    guard.cancel()


def main():
    a = parse()
    if a.impl == "reference":
        from baseline.run_reference import run_reference
        run_reference(a)
        return
    if not torch.cuda.is_available():
        print(json.dumps({"impl": "b200fw", "unavailable": "no CUDA device"}))
        return
    run_ours(a)


if __name__ == "__main__":
    main()
