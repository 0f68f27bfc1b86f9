#!/usr/bin/env python
"""Standalone inference with the paged engine.

    python scripts/run_inference.py --model-preset qwen3-0.6b --mode kv_cache --num-prompts 8 --max-tokens 64

CLI after the reference's (scripts/run_inference.py:39-60); YAML keys as in configs/inference/standalone.yaml.
"""
import argparse
import json
import os
import random
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

from b200fw.config import get_nested, load_yaml_config  # noqa: E402
from b200fw.infer import InferenceConfig, InferenceEngine  # noqa: E402
from b200fw.model import PRESETS, read_hf_config  # noqa: E402


def parse_args(argv=None):
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--config", default=None)
    ap.add_argument("--model-path", default="")
    ap.add_argument("--model-preset", default=None)
    ap.add_argument("--mode", choices=["kv_cache", "eager", "mock"], default=None)
    ap.add_argument("--prompt", action="append", default=None, help="text prompt (byte-level tokens without a tokenizer)")
    ap.add_argument("--num-prompts", type=int, default=4)
    ap.add_argument("--prompt-len", type=int, default=128)
    ap.add_argument("--max-tokens", type=int, default=None)
    ap.add_argument("--temperature", type=float, default=None)
    ap.add_argument("--top-p", type=float, default=None)
    ap.add_argument("--num-blocks", type=int, default=None)
    ap.add_argument("--kv-cache-dtype", choices=["fp16", "fp8"], default=None)
    ap.add_argument("--cuda-graph", action="store_true", default=None)
    ap.add_argument("--radix-cache", action="store_true", default=None)
    ap.add_argument("--partitioned-attention", action="store_true", default=None)
    ap.add_argument("--speculative", action="store_true", default=None)
    ap.add_argument("--seed", type=int, default=0)
    return ap.parse_args(argv)


def create_inference_config(a, y) -> InferenceConfig:
    pick = lambda cli, path, default: cli if cli is not None else get_nested(y, path, default)
    preset = a.model_preset or get_nested(y, "model.preset")
    path = a.model_path or get_nested(y, "model.name_or_path", "")
    mc = PRESETS[preset] if preset else read_hf_config(path)
    kw = dict(
        inference_mode=pick(a.mode, "inference.mode", "kv_cache"), model_path="" if preset else path,
        temperature=pick(a.temperature, "sampling.temperature", 0.7), top_p=pick(a.top_p, "sampling.top_p", 0.9),
        kv_cache_dtype=pick(a.kv_cache_dtype, "kv_cache.dtype", "fp16"), block_size=get_nested(y, "kv_cache.block_size", 16),
        max_num_batched_tokens=get_nested(y, "scheduler.max_num_batched_tokens", 8192),
        max_num_sequences=get_nested(y, "scheduler.max_num_sequences", 256),
        max_prefill_tokens=get_nested(y, "scheduler.max_prefill_tokens", 4096),
        chunk_size=get_nested(y, "scheduler.chunk_size", 512),
        enable_cuda_graph=bool(pick(a.cuda_graph, "optimizations.cuda_graph", False)),
        use_radix_cache=bool(pick(a.radix_cache, "optimizations.radix_cache", False)),
        enable_prefix_caching=bool(pick(a.radix_cache, "optimizations.prefix_caching", False)),
        enable_partitioned_attention=bool(pick(a.partitioned_attention, "optimizations.partitioned_attention", False)),
        attention_partition_size=get_nested(y, "optimizations.partition_size", 512),
        speculative_enabled=bool(pick(a.speculative, "speculative.enabled", False)),
        speculative_num_tokens=get_nested(y, "speculative.num_tokens", 4), seed=a.seed)
    nb = pick(a.num_blocks, "kv_cache.num_blocks", None)
    if nb is None:
        nb = InferenceConfig.auto_from_device(mc.num_layers, mc.num_kv_heads, mc.head_dim, kv_cache_dtype=kw["kv_cache_dtype"]).num_blocks
    return InferenceConfig.from_model_config(mc, num_blocks=int(nb), **kw)


def main(argv=None):
    a = parse_args(argv)
    y = load_yaml_config(a.config)
    cfg = create_inference_config(a, y)
    eng = InferenceEngine(cfg).initialize()
    rng = random.Random(a.seed)
    if a.prompt:
        from b200fw.data import SimpleTokenizer
        tok = SimpleTokenizer()
        prompts = [[min(t, cfg.vocab_size - 1) for t in tok.encode(p)] for p in a.prompt]
    else:
        prompts = [[rng.randrange(3, cfg.vocab_size) for _ in range(a.prompt_len)] for _ in range(a.num_prompts)]
    max_tokens = a.max_tokens if a.max_tokens is not None else get_nested(y, "sampling.max_tokens", 64)
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    t0 = time.perf_counter()
    outs = eng.generate(prompts, max_tokens)
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    n = sum(len(o) for o in outs if o)
    print(json.dumps({"mode": cfg.inference_mode, "prompts": len(prompts), "generated_tokens": n, "seconds": dt,
                      "tokens_per_s": n / dt if dt > 0 else 0.0, "first_output": (outs[0] or [])[:16],
                      "stats": {k: v for k, v in eng.get_stats().items() if not isinstance(v, dict)}}, indent=2))


if __name__ == "__main__":
    main()
