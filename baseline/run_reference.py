"""Reference arm of ``bench.py``: the unmodified reference package, through its own public API.

The reference is installed once, offline, into ``baseline/_ref`` with
``python -m pip install --no-index --no-build-isolation --no-deps --find-links <wheel dir> --target
baseline/_ref <reference checkout>`` (dependency resolution fails without an index, hence ``--no-deps``).
This module only *drives* it: it writes a Hugging Face style directory (``config.json`` plus seeded
N(0, 0.02) weights under the HF key names) for the benchmark architecture, builds the reference's
``TrainEngine`` with the same parallel layout, and calls its ``sft_step`` with the same synthetic token
batches, timing on the device.  None of this framework's models, kernels or engine are on that path.
"""
from __future__ import annotations

import json
import os
import sys
import time

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")


def _unavailable(why: str):
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)


def _hf_config(preset) -> dict:
    return {
        "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "vocab_size": preset.vocab_size,
        "hidden_size": preset.hidden_size, "num_hidden_layers": preset.num_layers,
        "num_attention_heads": preset.num_heads, "num_key_value_heads": preset.num_kv_heads,
        "head_dim": preset.head_dim, "intermediate_size": preset.intermediate_size,
        "max_position_embeddings": preset.max_position_embeddings, "rms_norm_eps": preset.rms_norm_eps,
        "rope_theta": preset.rope_theta, "tie_word_embeddings": preset.tie_word_embeddings,
    }


def write_fake_hf_dir(path: str, preset, with_weights: bool) -> None:
    """config.json + model.safetensors.  ``with_weights``: every tensor seeded N(0, 0.02) (norms = 1);
    otherwise a one-element placeholder so that the reference's loader finds a file and keeps its own
    initialisation for every parameter (used for architectures too large to stage through a file)."""
    from safetensors.torch import save_file
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(_hf_config(preset), f)
    tensors = {}
    if with_weights:
        g = torch.Generator().manual_seed(0)
        H, D, I = preset.hidden_size, preset.head_dim, preset.intermediate_size

        def rnd(*shape):
            return torch.empty(*shape).normal_(0.0, 0.02, generator=g).to(torch.bfloat16)

        tensors["model.embed_tokens.weight"] = rnd(preset.vocab_size, H)
        if not preset.tie_word_embeddings:
            tensors["lm_head.weight"] = rnd(preset.vocab_size, H)
        else:
            tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()
        tensors["model.norm.weight"] = torch.ones(H, dtype=torch.bfloat16)
        for i in range(preset.num_layers):
            p = f"model.layers.{i}."
            tensors[p + "self_attn.q_proj.weight"] = rnd(preset.num_heads * D, H)
            tensors[p + "self_attn.k_proj.weight"] = rnd(preset.num_kv_heads * D, H)
            tensors[p + "self_attn.v_proj.weight"] = rnd(preset.num_kv_heads * D, H)
            tensors[p + "self_attn.o_proj.weight"] = rnd(H, preset.num_heads * D)
            tensors[p + "self_attn.q_norm.weight"] = torch.ones(D, dtype=torch.bfloat16)
            tensors[p + "self_attn.k_norm.weight"] = torch.ones(D, dtype=torch.bfloat16)
            tensors[p + "mlp.gate_proj.weight"] = rnd(I, H)
            tensors[p + "mlp.up_proj.weight"] = rnd(I, H)
            tensors[p + "mlp.down_proj.weight"] = rnd(H, I)
            tensors[p + "input_layernorm.weight"] = torch.ones(H, dtype=torch.bfloat16)
            tensors[p + "post_attention_layernorm.weight"] = torch.ones(H, dtype=torch.bfloat16)
    else:
        tensors["placeholder"] = torch.zeros(1)
    save_file(tensors, os.path.join(path, "model.safetensors"))


def run_reference(a) -> None:
    if not os.path.isdir(os.path.join(REF, "src")):
        return _unavailable("reference is not installed under baseline/_ref")
    if not torch.cuda.is_available():
        return _unavailable("no CUDA device")
    sys.path.insert(0, REF)
    root = os.path.dirname(HERE)
    sys.path.insert(0, root)
    from b200fw.model.config import PRESETS   # architecture numbers only (a dataclass of ints)
    import copy
    preset = copy.deepcopy(PRESETS[a.model])
    if getattr(a, "layers", 0) > 0:
        preset.num_layers = a.layers        # smoke runs of a large architecture; not a benchmark config
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dp = world // (a.tp * a.pp)
    # ---- fake HF directory (rank 0 writes, the others wait for the marker file) -----------------------
    hf_dir = f"/tmp/b200fw_ref_hf_{a.model}" + (f"_L{a.layers}" if getattr(a, "layers", 0) > 0 else "")
    marker = os.path.join(hf_dir, ".ready")
    if rank == 0 and not os.path.exists(marker):
        write_fake_hf_dir(hf_dir, preset, with_weights=preset.num_params() < 5e9)
        open(marker, "w").close()
    t0 = time.time()
    while not os.path.exists(marker):
        if time.time() - t0 > 900:
            return _unavailable("timed out waiting for the synthetic HF directory")
        time.sleep(0.5)
    try:
        from src.engines.train_engine import TrainConfig, TrainEngine
    except Exception as e:  # noqa: BLE001
        return _unavailable(f"reference import failed: {type(e).__name__}: {e}")
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29511")
    cfg = TrainConfig(
        model_path=hf_dir, tp_size=a.tp, dp_size=dp, pp_size=a.pp,
        num_micro_batches=max(a.pp, a.grad_accum) if a.pp > 1 else 1, max_seq_len=a.seq_len,
        use_flash_attn=True, attention_backend="flash_attn", use_gradient_checkpoint=a.grad_ckpt,
        lora_rank=a.lora_rank, learning_rate=1e-5, gradient_accumulation_steps=a.grad_accum if a.pp == 1 else 1,
        grpo_beta=0.0, zero_stage=a.zero_stage, use_amp=True, amp_dtype="bf16", warmup_steps=2,
        total_training_steps=a.steps + a.warmup + 8)
    try:
        eng = TrainEngine(cfg)
        eng.initialize()
    except Exception as e:  # noqa: BLE001
        return _unavailable(f"reference TrainEngine.initialize failed: {type(e).__name__}: {str(e)[:200]}")
    dev = torch.device("cuda", local)
    dp_rank = getattr(eng.parallel_ctx, "dp_rank", 0)
    g = torch.Generator().manual_seed(1234 + dp_rank)
    micro_per_step = a.grad_accum if a.pp == 1 else 1
    batches = []
    for _ in range(micro_per_step * 2):
        ids = torch.randint(0, preset.vocab_size, (a.micro_batch, a.seq_len), generator=g)
        half = a.seq_len // 2
        batches.append(([r[:half].tolist() for r in ids], [r[half:].tolist() for r in ids]))

    def barrier():
        if world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize()

    try:
        for k in range(a.warmup * micro_per_step):
            eng.sft_step(*batches[k % len(batches)])
        barrier()
        from bench import ClockSampler
        sampler = ClockSampler(local)
        if rank == 0:
            sampler.start()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        loss = 0.0
        for k in range(a.steps * micro_per_step):
            loss = eng.sft_step(*batches[k % len(batches)]).loss
        e.record()
        barrier()
    except Exception as e2:  # noqa: BLE001
        return _unavailable(f"reference sft_step failed: {type(e2).__name__}: {str(e2)[:200]}")
    ms = s.elapsed_time(e)
    if world > 1:
        import torch.distributed as dist
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t)
    clocks = sampler.stop() if rank == 0 else None
    tokens_per_step = a.micro_batch * a.seq_len * micro_per_step * dp
    tps = tokens_per_step * a.steps / (ms * 1e-3)
    if rank == 0:
        print(json.dumps({
            "metric": "sft_tokens_per_s", "value": tps, "unit": "tokens/s", "n_gpus": world, "steps": a.steps,
            "warmup": a.warmup, "ms_per_step": ms / a.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic (seeded uniform tokens, random-init weights)",
            "impl": "reference",
            "config": {"model": (f"{a.model}-arch full SFT" if a.lora_rank <= 0 else f"{a.model}-arch LoRA r{a.lora_rank}")
                       + (f" (layers cut to {a.layers}: smoke run, not the named config)" if getattr(a, "layers", 0) > 0 else ""),
                       "grad_ckpt": a.grad_ckpt,
                       "global_batch": a.micro_batch * micro_per_step * dp, "micro_batch_per_gpu": a.micro_batch,
                       "grad_accum": a.grad_accum, "seq_len": a.seq_len,
                       "parallelism": f"dp{dp}" + (f"+tp{a.tp}" if a.tp > 1 else "") + (f"+pp{a.pp}" if a.pp > 1 else ""),
                       "zero_stage": a.zero_stage, "attention_backend": "flash_attn",
                       "api": "src.engines.train_engine.TrainEngine.sft_step (token lists in, loss.item() out)"},
            "e2e": {"value": tps, "unit": "tokens/s", "note": "the reference's public step takes host token lists and reads the loss back, so its only number is end to end"},
            "final_loss": loss, "gpu_launches": 0, "clocks": clocks,
        }), flush=True)
