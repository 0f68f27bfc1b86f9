#!/usr/bin/env python
"""Reference arms for the metrics that are not a training step: decode tokens/s, GRPO iteration seconds and
weight-sync milliseconds, each through the unmodified reference package's own public API (installed under
``baseline/_ref``; nothing of this framework's models, kernels or engines runs here).

    python baseline/run_reference_extras.py decode [--requests 256 --prompt-min 128 --prompt-max 1024 --max-tokens 256]
        src.inference.engine.InferenceEngine(inference_mode="kv_cache").generate(token lists) on a synthetic
        Qwen3-0.6B HF directory (config.json, seeded weights, a minimal tokenizer.json)
    python baseline/run_reference_extras.py grpo [--prompts 64 --num-samples 8 --prompt-len 256 --max-tokens 512]
        src.engines.train_engine.TrainEngine.generate (its "custom" rollout path: no KV cache, one sequence at a
        time) timed on a few sequences, and TrainEngine.grpo_step on the largest batch that fits
    torchrun --nproc-per-node 2 baseline/run_reference_extras.py sync
        src.transfer.nccl_transfer.NCCLWeightTransfer.broadcast_weights / receive_weights of the 0.6B state dict

Each sub-command prints one JSON line on rank 0.  An arm that cannot run prints the exception text it stopped on
under ``"unavailable"`` and exits 0: the record of why is the result.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
import traceback

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
REF = os.path.join(HERE, "_ref")
sys.path.insert(0, ROOT)
sys.path.insert(0, REF)

from baseline.run_reference import write_fake_hf_dir  # noqa: E402
from b200fw.model.config import PRESETS  # noqa: E402  (architecture numbers only)
from b200fw.obs.clocks import ClockSampler  # noqa: E402  (nvidia-smi sampler, no kernels)


def emit(d):
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps(d), flush=True)


def hf_dir_for(model: str, with_tokenizer: bool = False) -> str:
    """Synthetic HF directory (rank 0 writes; other ranks wait for the marker)."""
    preset = PRESETS[model]
    path = f"/tmp/b200fw_ref_hf_{model}"
    marker = os.path.join(path, ".ready")
    if int(os.environ.get("RANK", "0")) == 0:
        if not os.path.exists(marker):
            write_fake_hf_dir(path, preset, with_weights=True)
            open(marker, "w").close()
        if with_tokenizer and not os.path.exists(os.path.join(path, "tokenizer.json")):
            write_minimal_tokenizer(path, preset.vocab_size)
    t0 = time.time()
    while not os.path.exists(marker) and time.time() - t0 < 900:
        time.sleep(0.5)
    return path


def write_minimal_tokenizer(path: str, vocab_size: int) -> None:
    """A word-level ``tokenizer.json`` with one entry per id: enough for ``AutoTokenizer.from_pretrained``;
    the benchmark passes token ids, so no text is ever tokenised."""
    from tokenizers import Tokenizer
    from tokenizers.models import WordLevel
    from tokenizers.pre_tokenizers import Whitespace
    vocab = {f"t{i}": i for i in range(vocab_size)}
    tok = Tokenizer(WordLevel(vocab, unk_token="t0"))
    tok.pre_tokenizer = Whitespace()
    tok.save(os.path.join(path, "tokenizer.json"))
    with open(os.path.join(path, "tokenizer_config.json"), "w") as f:
        json.dump({"tokenizer_class": "PreTrainedTokenizerFast", "unk_token": "t0", "eos_token": "t2",
                   "pad_token": "t0", "model_max_length": 40960}, f)
    with open(os.path.join(path, "generation_config.json"), "w") as f:
        json.dump({"eos_token_id": 2, "pad_token_id": 0}, f)


def decode_workload(vocab, requests, pmin, pmax, group, shared, seed=0):
    """Prompt lengths uniform in [pmin, pmax]; each group of ``group`` requests shares its first ``shared`` tokens."""
    g = torch.Generator().manual_seed(seed)
    prompts = []
    for i in range(requests):
        if i % group == 0:
            prefix = torch.randint(3, vocab, (shared,), generator=g).tolist()
        n = int(torch.randint(pmin, pmax + 1, (1,), generator=g))
        tail = torch.randint(3, vocab, (max(0, n - shared),), generator=g).tolist()
        prompts.append((prefix + tail)[:max(n, 1)] if n <= shared else prefix + tail)
    return prompts


def run_decode(a):
    torch.cuda.set_device(0)
    path = hf_dir_for(a.model, with_tokenizer=True)
    preset = PRESETS[a.model]
    try:
        from src.inference.engine import InferenceConfig, InferenceEngine
    except Exception as e:  # noqa: BLE001
        return emit({"impl": "reference", "metric": "decode_tokens_per_s", "unavailable": f"import failed: {type(e).__name__}: {e}"})
    prompts = decode_workload(preset.vocab_size, a.requests, a.prompt_min, a.prompt_max, 8, 512)
    blocks = sum((len(p) + a.max_tokens + 15) // 16 + 1 for p in prompts) + 64
    cfg = InferenceConfig(num_layers=preset.num_layers, num_heads=preset.num_heads, num_kv_heads=preset.num_kv_heads,
                          head_dim=preset.head_dim, hidden_size=preset.hidden_size, vocab_size=preset.vocab_size,
                          num_blocks=blocks, block_size=16, max_num_batched_tokens=8192, max_num_sequences=a.requests,
                          chunk_size=512, enable_prefix_caching=True, use_radix_cache=True, temperature=0.8, top_p=0.95,
                          inference_mode="kv_cache", model_path=path, dtype="bfloat16")
    try:
        eng = InferenceEngine(cfg)
        eng.initialize()
    except Exception as e:  # noqa: BLE001
        return emit({"impl": "reference", "metric": "decode_tokens_per_s",
                     "unavailable": f"InferenceEngine.initialize failed: {type(e).__name__}: {str(e)[:400]}",
                     "trace_tail": traceback.format_exc()[-600:]})
    # The reference's engine prefills one sequence at a time and runs its decode loop in Python: the named workload
    # (256 requests x 256 tokens) may take far longer than a benchmark slot.  Run growing slices of it while the
    # projected time of the next one fits the budget, and report the largest slice that ran.
    ladder = [(8, 16), (32, 64), (64, 128), (a.requests, a.max_tokens)]
    budget_s, done, last = a.budget_s, [], None
    sampler = ClockSampler(0)
    sampler.start()
    try:
        eng.generate(prompts[:2], max_tokens=4, temperature=0.8)                  # lazy initialisation
        torch.cuda.synchronize()
        for n_req, n_tok in ladder:
            n_req, n_tok = min(n_req, a.requests), min(n_tok, a.max_tokens)
            if last is not None:
                projected = last["seconds_wall"] * (n_req * n_tok) / (last["requests"] * last["max_tokens"])
                if projected > budget_s:
                    done.append({"requests": n_req, "max_tokens": n_tok, "skipped": f"projected {projected:.0f} s > budget {budget_s:.0f} s"})
                    continue
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            t0 = time.perf_counter()
            outs = eng.generate(prompts[:n_req], max_tokens=n_tok, temperature=0.8)
            e.record()
            torch.cuda.synchronize()
            wall = time.perf_counter() - t0
            if outs is None:
                done.append({"requests": n_req, "max_tokens": n_tok, "error": "generate returned None (its CUDA OOM recovery path)"})
                break
            n_out = sum(len(o) for o in outs)
            last = {"requests": n_req, "max_tokens": n_tok, "prompt_tokens": sum(len(p) for p in prompts[:n_req]),
                    "output_tokens": n_out, "seconds_device": s.elapsed_time(e) * 1e-3, "seconds_wall": wall,
                    "output_tokens_per_s": n_out / (s.elapsed_time(e) * 1e-3)}
            done.append(last)
    except Exception as e2:  # noqa: BLE001
        return emit({"impl": "reference", "metric": "decode_tokens_per_s", "slices": done,
                     "unavailable": f"InferenceEngine.generate failed: {type(e2).__name__}: {str(e2)[:400]}",
                     "trace_tail": traceback.format_exc()[-600:]})
    clocks = sampler.stop()
    if last is None:
        return emit({"impl": "reference", "metric": "decode_tokens_per_s", "slices": done, "unavailable": "no slice of the workload ran"})
    emit({"impl": "reference", "metric": "generation_output_tokens_per_s", "value": last["output_tokens_per_s"], "unit": "tokens/s",
          "largest_slice_that_ran": last, "slices": done, "named_workload": {"requests": a.requests, "max_tokens": a.max_tokens},
          "api": "src.inference.engine.InferenceEngine.generate (inference_mode=kv_cache); prefill and decode are "
                 "not separable through its API, so this is output tokens over the whole call",
          "clocks": clocks})


def run_grpo(a):
    torch.cuda.set_device(0)
    path = hf_dir_for(a.model)
    preset = PRESETS[a.model]
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29513")
    try:
        from src.engines.train_engine import TrainConfig, TrainEngine
        cfg = TrainConfig(model_path=path, tp_size=1, dp_size=1, pp_size=1, max_seq_len=a.prompt_len + a.max_tokens,
                          use_flash_attn=True, attention_backend="flash_attn", lora_rank=0, learning_rate=1e-6,
                          gradient_accumulation_steps=1, grpo_num_samples=a.num_samples, grpo_beta=0.01,
                          grpo_clip_eps=0.2, zero_stage=1, use_amp=True, amp_dtype="bf16", warmup_steps=0,
                          total_training_steps=100)
        eng = TrainEngine(cfg)
        eng.initialize()
    except Exception as e:  # noqa: BLE001
        return emit({"impl": "reference", "metric": "grpo_iteration_s",
                     "unavailable": f"TrainEngine.initialize failed: {type(e).__name__}: {str(e)[:400]}"})
    g = torch.Generator().manual_seed(0)
    out = {"impl": "reference", "metric": "grpo_iteration_s", "config": {
        "prompts": a.prompts, "num_samples": a.num_samples, "prompt_len": a.prompt_len, "max_tokens": a.max_tokens}}
    sampler = ClockSampler(0)
    sampler.start()
    # ---- rollout: the reference's own sampler, TrainEngine.generate (no KV cache, one sequence at a time) -------
    try:
        prompt = torch.randint(3, preset.vocab_size, (a.prompt_len,), generator=g).tolist()
        eng.generate(prompt, max_new_tokens=4, temperature=0.8, top_p=0.95)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        n_tok = 0
        for _ in range(a.rollout_samples):
            n_tok += len(eng.generate(prompt, max_new_tokens=a.rollout_tokens, temperature=0.8, top_p=0.95))
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        per_tok = dt / max(1, n_tok)
        # the cost of a token grows with the sequence (full re-forward): the first rollout_tokens of a response are
        # its cheapest, so scaling this figure to max_tokens under-estimates the reference's rollout time
        out["rollout"] = {"sequences_timed": a.rollout_samples, "tokens_timed": n_tok, "seconds": dt,
                          "seconds_per_token": per_tok,
                          "iteration_estimate_s": per_tok * a.prompts * a.num_samples * a.max_tokens,
                          "note": "lower bound: measured on the first tokens of a response, full re-forward per token"}
    except Exception as e:  # noqa: BLE001
        out["rollout"] = {"unavailable": f"{type(e).__name__}: {str(e)[:300]}"}
    # ---- train: grpo_step at the named batch, then smaller ones until one fits -----------------------------
    tries, n = [], a.prompts
    while n >= 1:
        P = [torch.randint(3, preset.vocab_size, (a.prompt_len,), generator=g).tolist() for _ in range(n)]
        R = [[torch.randint(3, preset.vocab_size, (a.max_tokens,), generator=g).tolist() for _ in range(a.num_samples)]
             for _ in range(n)]
        W = [[float(torch.rand(1, generator=g)) for _ in range(a.num_samples)] for _ in range(n)]
        try:
            torch.cuda.synchronize()
            eng.grpo_step(P, R, W)                           # warm-up of this shape
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            for _ in range(2):
                m = eng.grpo_step(P, R, W)
            torch.cuda.synchronize()
            dt = (time.perf_counter() - t0) / 2
            tries.append({"prompts": n, "sequences": n * a.num_samples, "seconds_per_step": dt, "loss": float(m.loss)})
            break
        except Exception as e:  # noqa: BLE001 - typically torch.OutOfMemoryError from the [B*K, S, V] logits
            tries.append({"prompts": n, "sequences": n * a.num_samples,
                          "error": f"{type(e).__name__}: {str(e)[:240]}"})
            eng.optimizer.zero_grad()
            del P, R, W
            import gc
            gc.collect()
            torch.cuda.empty_cache()
            n //= 2
    out["train"] = tries
    ok = [t for t in tries if "seconds_per_step" in t]
    if ok and "seconds_per_token" in out.get("rollout", {}):
        chunks = -(-a.prompts // ok[0]["prompts"])
        out["train_iteration_estimate_s"] = ok[0]["seconds_per_step"] * chunks
        out["value"] = out["rollout"]["iteration_estimate_s"] + out["train_iteration_estimate_s"]
        out["unit"] = "s (rollout estimate + train: the reference has no batched sampler of its own to time whole)"
    out["clocks"] = sampler.stop()
    emit(out)


def run_sync(a):
    import torch.distributed as dist
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world < 2:
        return emit({"impl": "reference", "metric": "weight_sync_ms", "unavailable": "needs at least 2 ranks (torchrun)"})
    dist.init_process_group("nccl")
    try:
        from src.transfer.nccl_transfer import NCCLWeightTransfer
    except Exception as e:  # noqa: BLE001
        return emit({"impl": "reference", "metric": "weight_sync_ms", "unavailable": f"import failed: {type(e).__name__}: {e}"})
    preset = PRESETS[a.model]
    H, D, I = preset.hidden_size, preset.head_dim, preset.intermediate_size
    shapes = {"model.embed_tokens.weight": (preset.vocab_size, H), "model.norm.weight": (H,)}
    for i in range(preset.num_layers):
        p = f"model.layers.{i}."
        shapes.update({p + "self_attn.q_proj.weight": (preset.num_heads * D, H), p + "self_attn.k_proj.weight": (preset.num_kv_heads * D, H),
                       p + "self_attn.v_proj.weight": (preset.num_kv_heads * D, H), p + "self_attn.o_proj.weight": (H, preset.num_heads * D),
                       p + "self_attn.q_norm.weight": (D,), p + "self_attn.k_norm.weight": (D,),
                       p + "mlp.gate_proj.weight": (I, H), p + "mlp.up_proj.weight": (I, H), p + "mlp.down_proj.weight": (H, I),
                       p + "input_layernorm.weight": (H,), p + "post_attention_layernorm.weight": (H,)})
    sd = {k: torch.full(s, 0.01 * (rank == 0), dtype=torch.bfloat16, device="cuda") for k, s in shapes.items()}
    nbytes = sum(t.numel() * 2 for t in sd.values())
    tr = NCCLWeightTransfer(src_rank=0)
    times = []
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    try:
        for it in range(a.warmup + a.iters):
            dist.barrier()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            if rank == 0:
                tr.broadcast_weights(sd)
            else:
                tr.receive_weights(sd)
            torch.cuda.synchronize()
            dt = torch.tensor([time.perf_counter() - t0], dtype=torch.float64, device="cuda")
            dist.all_reduce(dt, op=dist.ReduceOp.MAX)
            if it >= a.warmup:
                times.append(float(dt) * 1e3)
    except Exception as e:  # noqa: BLE001
        return emit({"impl": "reference", "metric": "weight_sync_ms", "unavailable": f"{type(e).__name__}: {str(e)[:300]}"})
    clocks = sampler.stop() if rank == 0 else None
    times.sort()
    ok = bool(rank == 0 or abs(float(sd["model.norm.weight"][0]) - 0.01) < 1e-3)
    emit({"impl": "reference", "metric": "weight_sync_ms", "value": times[len(times) // 2], "unit": "ms", "best_ms": times[0],
          "bytes": nbytes, "gbs": nbytes / (times[len(times) // 2] * 1e-3) / 1e9, "ranks": world, "tensors": len(sd),
          "received_ok": ok, "api": "src.transfer.nccl_transfer.NCCLWeightTransfer.broadcast_weights / receive_weights "
          "(includes its per-sync checksum and object broadcasts; max over ranks, host clock around a device sync)",
          "clocks": clocks})
    dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("what", choices=["decode", "grpo", "sync"])
    ap.add_argument("--model", default="qwen3-0.6b")
    ap.add_argument("--requests", type=int, default=256)
    ap.add_argument("--prompt-min", type=int, default=128)
    ap.add_argument("--prompt-max", type=int, default=1024)
    ap.add_argument("--max-tokens", type=int, default=None)
    ap.add_argument("--prompts", type=int, default=64)
    ap.add_argument("--num-samples", type=int, default=8)
    ap.add_argument("--prompt-len", type=int, default=256)
    ap.add_argument("--rollout-samples", type=int, default=2)
    ap.add_argument("--rollout-tokens", type=int, default=32)
    ap.add_argument("--budget-s", type=float, default=150.0, help="decode: skip a slice whose projected time exceeds this")
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=2)
    a = ap.parse_args()
    if a.max_tokens is None:
        a.max_tokens = 256 if a.what == "decode" else 512
    if not os.path.isdir(os.path.join(REF, "src")):
        return emit({"impl": "reference", "unavailable": "reference is not installed under baseline/_ref"})
    if not torch.cuda.is_available():
        return emit({"impl": "reference", "unavailable": "no CUDA device"})
    {"decode": run_decode, "grpo": run_grpo, "sync": run_sync}[a.what](a)


if __name__ == "__main__":
    main()
