#!/usr/bin/env python
"""Standalone inference with the paged engine.

    python scripts/run_inference.py --model-preset qwen3-0.6b --mode kv_cache --num-prompts 8 --max-tokens 64
    python scripts/run_inference.py -m /path/to/Qwen3-0.6B --mode kv_cache -p "What is 2+2?" --num-samples 4 -o out.jsonl
    python scripts/run_inference.py -m /path/to/Qwen3-0.6B -i prompts.jsonl --batch-size 32 --enable-prefix-cache
    python scripts/run_inference.py --model-preset tiny128 --interactive

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
    ap.add_argument("--config", default=None, help="YAML file (configs/inference/standalone.yaml schema)")
    ap.add_argument("--model", "-m", "--model-path", dest="model_path", default="", help="HF model directory")
    ap.add_argument("--model-preset", default=None, help="random-init architecture preset instead of a directory")
    ap.add_argument("--mode", choices=["kv_cache", "eager", "mock"], default=None)
    ap.add_argument("--prompt", "-p", action="append", default=None, help="text prompt (repeatable)")
    ap.add_argument("--input", "-i", default=None, help="JSONL file: one string or {\"prompt\"|\"text\": ...} per line")
    ap.add_argument("--output", "-o", default=None, help="write one JSON record per sample to this JSONL file")
    ap.add_argument("--interactive", action="store_true", help="read prompts from stdin until 'quit'")
    ap.add_argument("--num-samples", type=int, default=1, help="samples per prompt")
    ap.add_argument("--batch-size", type=int, default=0, help="prompts per generate() call (0: all at once)")
    ap.add_argument("--num-prompts", type=int, default=4, help="synthetic prompts when no text prompt is given")
    ap.add_argument("--prompt-len", type=int, default=128)
    ap.add_argument("--max-tokens", type=int, default=None)
    ap.add_argument("--temperature", type=float, default=None)
    ap.add_argument("--top-p", type=float, default=None)
    ap.add_argument("--num-blocks", type=int, default=None)
    ap.add_argument("--block-size", type=int, default=None)
    ap.add_argument("--kv-cache-dtype", choices=["fp16", "fp8"], default=None)
    ap.add_argument("--cuda-graph", "--enable-cuda-graph", dest="cuda_graph", action="store_true", default=None)
    ap.add_argument("--radix-cache", action="store_true", default=None)
    ap.add_argument("--enable-prefix-cache", dest="prefix_cache", action="store_true", default=None)
    ap.add_argument("--enable-async", dest="async_scheduling", action="store_true", default=None,
                    help="accepted for compatibility: the engine always interleaves prefill chunks and decode")
    ap.add_argument("--partitioned-attention", "--enable-partitioned-attn", dest="partitioned_attention",
                    action="store_true", default=None)
    ap.add_argument("--speculative", action="store_true", default=None)
    ap.add_argument("--seed", type=int, default=0)
    return ap.parse_args(argv)


def _first(y, paths, default=None):
    for path in paths:
        v = get_nested(y, path)
        if v is not None:
            return v
    return default


def create_inference_config(a, y) -> InferenceConfig:
    """CLI over YAML over defaults.  The YAML may use this repository's keys (configs/inference/standalone.yaml) or the
    reference's (``model.path``, ``inference.temperature``, ``kv_cache.enable_cuda_graph``, ``advanced.*``)."""
    def pick(cli, paths, default):
        return cli if cli is not None else _first(y, paths if isinstance(paths, (list, tuple)) else [paths], default)

    preset = a.model_preset or get_nested(y, "model.preset")
    path = a.model_path or _first(y, ["model.name_or_path", "model.path"], "")
    mc = PRESETS[preset] if preset else read_hf_config(path)
    radix = pick(a.radix_cache, ["optimizations.radix_cache", "advanced.use_radix_cache"], False)
    kw = dict(
        inference_mode=pick(a.mode, "inference.mode", "kv_cache"), model_path="" if preset else path,
        temperature=pick(a.temperature, ["sampling.temperature", "inference.temperature"], 0.7),
        top_p=pick(a.top_p, ["sampling.top_p", "inference.top_p"], 0.9),
        kv_cache_dtype=pick(a.kv_cache_dtype, "kv_cache.dtype", "fp16"),
        block_size=int(pick(a.block_size, "kv_cache.block_size", 16)),
        enable_async_scheduling=bool(pick(a.async_scheduling, ["optimizations.async_scheduling",
                                                               "advanced.enable_async_scheduling"], False)),
        max_num_batched_tokens=get_nested(y, "scheduler.max_num_batched_tokens", 8192),
        max_num_sequences=get_nested(y, "scheduler.max_num_sequences", 256),
        max_prefill_tokens=get_nested(y, "scheduler.max_prefill_tokens", 4096),
        chunk_size=get_nested(y, "scheduler.chunk_size", 512),
        enable_cuda_graph=bool(pick(a.cuda_graph, ["optimizations.cuda_graph", "kv_cache.enable_cuda_graph"], False)),
        use_radix_cache=bool(radix),
        enable_prefix_caching=bool(a.prefix_cache or radix or _first(y, ["optimizations.prefix_caching",
                                                                         "kv_cache.enable_prefix_caching"], False)),
        enable_prefix_reuse=bool(_first(y, ["optimizations.prefix_reuse", "kv_cache.enable_prefix_reuse"], True)),
        enable_partitioned_attention=bool(pick(a.partitioned_attention, ["optimizations.partitioned_attention",
                                                                         "advanced.enable_partitioned_attention"], False)),
        attention_partition_size=get_nested(y, "optimizations.partition_size", 512),
        speculative_enabled=bool(pick(a.speculative, "speculative.enabled", False)),
        speculative_num_tokens=get_nested(y, "speculative.num_tokens", 4), seed=a.seed)
    nb = pick(a.num_blocks, "kv_cache.num_blocks", None)
    if nb is None:
        nb = InferenceConfig.auto_from_device(mc.num_layers, mc.num_kv_heads, mc.head_dim, kv_cache_dtype=kw["kv_cache_dtype"]).num_blocks
    return InferenceConfig.from_model_config(mc, num_blocks=int(nb), **kw)


def load_prompts_from_file(path: str):
    """JSONL: each line a JSON string or an object with a ``prompt`` (or ``text``) field."""
    prompts = []
    with open(path) as f:
        for line in f:
            line = line.strip()
            if not line:
                continue
            d = json.loads(line)
            prompts.append(d if isinstance(d, str) else d.get("prompt", d.get("text", "")))
    return prompts


def _sync():
    if torch.cuda.is_available():
        torch.cuda.synchronize()


def generate_text(eng, tok, prompts, a, max_tokens, vocab):
    """``num_samples`` answers per text prompt, ``batch_size`` prompts per engine call; one record per sample."""
    results = []
    step = a.batch_size if a.batch_size > 0 else max(1, len(prompts))
    for s in range(0, len(prompts), step):
        chunk = prompts[s:s + step]
        toks = [[min(t, vocab - 1) for t in tok.encode(p)] for p in chunk]
        empty = [p for p, t in zip(chunk, toks) if not t]
        if empty:       # a prompt that encodes to nothing cannot be served: report it and go on with the others
            print(f"[run_inference] {len(empty)} empty prompt(s) skipped", file=sys.stderr)
            for p in empty:
                results.append({"prompt": p, "sample_idx": 0, "output": "", "num_tokens": 0, "time_s": 0.0,
                                "tokens_per_s": 0.0, "error": "empty prompt"})
            chunk, toks = [p for p, t in zip(chunk, toks) if t], [t for t in toks if t]
            if not chunk:
                continue
        batch = [t for t in toks for _ in range(a.num_samples)]
        _sync()
        t0 = time.perf_counter()
        outs = eng.generate(batch, max_tokens, a.temperature, a.top_p)
        _sync()
        dt = time.perf_counter() - t0
        for j, p in enumerate(chunk):
            for k in range(a.num_samples):
                o = outs[j * a.num_samples + k] or []
                results.append({"prompt": p, "sample_idx": k, "output": tok.decode(o, skip_special_tokens=True),
                                "num_tokens": len(o), "time_s": round(dt, 3),
                                "tokens_per_s": round(sum(len(x or []) for x in outs) / dt, 1) if dt > 0 else 0.0})
    return results


def run_interactive(eng, tok, a, max_tokens, vocab, stdin=None, out=print):
    stdin = stdin if stdin is not None else sys.stdin
    out("interactive mode: one prompt per line, 'quit' to leave")
    while True:
        line = stdin.readline()
        if not line or line.strip().lower() in ("quit", "exit", "q"):
            break
        if not line.strip():
            continue
        for r in generate_text(eng, tok, [line.strip()], a, max_tokens, vocab):
            out(f"[{r['num_tokens']} tokens, {r['tokens_per_s']} tok/s] {r['output']}")


def main(argv=None):
    a = parse_args(argv)
    y = load_yaml_config(a.config)
    cfg = create_inference_config(a, y)
    eng = InferenceEngine(cfg).initialize()
    max_tokens = a.max_tokens if a.max_tokens is not None else _first(y, ["sampling.max_tokens", "inference.max_tokens"], 64)
    if a.num_samples == 1:
        a.num_samples = int(get_nested(y, "inference.num_samples", 1))
    if a.batch_size == 0:
        a.batch_size = int(get_nested(y, "inference.batch_size", 0))
    from b200fw.data.pipeline import _load_tokenizer
    tok = _load_tokenizer(a.model_path or None)          # the model directory's tokenizer, else byte-level
    if a.interactive:
        run_interactive(eng, tok, a, max_tokens, cfg.vocab_size)
        return
    texts = list(a.prompt or []) + (load_prompts_from_file(a.input) if a.input else [])
    if texts:
        results = generate_text(eng, tok, texts, a, max_tokens, cfg.vocab_size)
        if a.output:
            with open(a.output, "w") as f:
                for r in results:
                    f.write(json.dumps(r, ensure_ascii=False) + "\n")
        n = sum(r["num_tokens"] for r in results)
        print(json.dumps({"mode": cfg.inference_mode, "prompts": len(texts), "samples": len(results),
                          "generated_tokens": n, "output": a.output,
                          "first_output": results[0]["output"][:200] if results else ""}, indent=2, ensure_ascii=False))
        return
    rng = random.Random(a.seed)
    prompts = [[rng.randrange(3, cfg.vocab_size) for _ in range(a.prompt_len)] for _ in range(a.num_prompts)]
    _sync()
    t0 = time.perf_counter()
    outs = eng.generate(prompts, max_tokens)
    _sync()
    dt = time.perf_counter() - t0
    n = sum(len(o) for o in outs if o)
    print(json.dumps({"mode": cfg.inference_mode, "prompts": len(prompts), "generated_tokens": n, "seconds": dt,
                      "tokens_per_s": n / dt if dt > 0 else 0.0, "first_output": (outs[0] or [])[:16],
                      "stats": {k: v for k, v in eng.get_stats().items() if not isinstance(v, dict)}}, indent=2))


if __name__ == "__main__":
    main()
