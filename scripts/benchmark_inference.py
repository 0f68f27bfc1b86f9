#!/usr/bin/env python
"""Inference benchmark of the paged engine: prefill ms, decode ms/token, decode tokens/s.

Default workload (the standalone-inference benchmark configuration): Qwen3-0.6B architecture with random
weights, 256 concurrent requests, prompt lengths uniform in [128, 1024], 256 output tokens each,
temperature 0.8 / top-p 0.95, every group of 8 requests sharing a 512-token prefix (radix cache), KV
blocks of 16 tokens in 16-bit or fp8.  Variants: --cuda-graph, --speculative, --long-context (one 32k
sequence, partitioned attention).  Timed with CUDA events around whole engine phases.
"""
import argparse
import json
import os
import random
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

from b200fw.infer import InferenceConfig, InferenceEngine  # noqa: E402
from b200fw.model import PRESETS, ParallelTransformerModel  # noqa: E402
from b200fw.obs.clocks import ClockSampler  # noqa: E402


def parse_args(argv=None):
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--model-preset", default="qwen3-0.6b")
    ap.add_argument("--num-requests", type=int, default=256)
    ap.add_argument("--min-prompt", type=int, default=128)
    ap.add_argument("--max-prompt", type=int, default=1024)
    ap.add_argument("--output-tokens", type=int, default=256)
    ap.add_argument("--shared-prefix", type=int, default=512)
    ap.add_argument("--group", type=int, default=8)
    ap.add_argument("--kv-cache-dtype", choices=["fp16", "fp8"], default="fp16")
    ap.add_argument("--token-budget", type=int, default=8192)
    ap.add_argument("--chunk-size", type=int, default=512)
    ap.add_argument("--cuda-graph", action="store_true")
    ap.add_argument("--no-radix", action="store_true")
    ap.add_argument("--speculative", action="store_true")
    ap.add_argument("--long-context", type=int, default=0, help="single sequence of this many prompt tokens")
    ap.add_argument("--temperature", type=float, default=0.8)
    ap.add_argument("--top-p", type=float, default=0.95)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--warmup", type=int, default=1)
    ap.add_argument("--profile-decode-steps", type=int, default=0,
                    help="bracket this many decode steps with cudaProfilerStart/Stop (for `ncu --profile-from-start off`)")
    ap.add_argument("--balance-splits", action="store_true",
                    help="split every sequence's keys over a few CTAs when the decode grid would fill only a few waves")
    ap.add_argument("--no-async-decode", dest="async_decode", action="store_false",
                    help="read every step's sampled ids back before the next step is launched")
    return ap.parse_args(argv)


def make_prompts(a, vocab):
    rng = random.Random(a.seed)
    if a.long_context:
        return [[rng.randrange(3, vocab) for _ in range(a.long_context)]]
    out, prefix = [], []
    for i in range(a.num_requests):
        if i % a.group == 0:
            prefix = [rng.randrange(3, vocab) for _ in range(a.shared_prefix)]
        n = rng.randint(a.min_prompt, a.max_prompt)
        body = [rng.randrange(3, vocab) for _ in range(max(1, n - len(prefix)))]
        out.append(prefix[:max(0, n - 1)] + body if n > len(prefix) else prefix[:n - 1] + body[:1])
    return out


def main(argv=None):
    a = parse_args(argv)
    assert torch.cuda.is_available(), "the inference benchmark needs a GPU"
    mc = PRESETS[a.model_preset]
    dev = torch.device("cuda", 0)
    model = ParallelTransformerModel(mc, dtype=torch.bfloat16, device=dev)
    model.init_weights(a.seed)
    for p in model.parameters():
        p.requires_grad_(False)
    prompts = make_prompts(a, mc.vocab_size)
    total_ctx = sum(len(p) for p in prompts) + len(prompts) * a.output_tokens
    blocks = total_ctx // 16 + 4 * len(prompts) + 1024
    cfg = InferenceConfig.from_model_config(
        mc, num_blocks=blocks, inference_mode="kv_cache", kv_cache_dtype=a.kv_cache_dtype,
        max_num_batched_tokens=a.token_budget, max_prefill_tokens=a.token_budget, chunk_size=a.chunk_size,
        max_num_sequences=max(256, len(prompts)), use_radix_cache=not a.no_radix, enable_prefix_caching=not a.no_radix,
        max_cached_blocks=blocks, enable_cuda_graph=a.cuda_graph, speculative_enabled=a.speculative,
        speculative_num_tokens=4, speculative_draft_layers=2, enable_partitioned_attention=bool(a.long_context),
        attention_partition_size=512, temperature=a.temperature, top_p=a.top_p, eos_token_id=None, seed=a.seed,
        adaptive_chunking=False, async_decode=a.async_decode,
        decode_balance_splits=a.balance_splits)
    eng = InferenceEngine(cfg, model).initialize()
    for _ in range(a.warmup):     # compile-free warm-up: allocator, graphs, tensor maps
        eng.generate(prompts[: min(8, len(prompts))], 8)
        eng.on_weights_updated()
    ev = lambda: torch.cuda.Event(enable_timing=True)
    # ---- prefill phase: add everything, step until every request has its first token -----------------------
    for i, p in enumerate(prompts):
        eng.add_request(f"b{i}", p, a.output_tokens)
    s0, s1, s2 = ev(), ev(), ev()
    sampler = ClockSampler(0)
    sampler.start()
    s0.record()
    steps_prefill = 0
    while any(r.num_generated_tokens == 0 for r in eng.requests.values()):
        eng.step()
        steps_prefill += 1
    s1.record()
    first = sum(r.num_generated_tokens for r in eng.requests.values())
    steps_decode = 0
    if a.profile_decode_steps:
        torch.cuda.synchronize()
        torch.cuda.profiler.start()
    while eng.has_pending():
        eng.step()
        steps_decode += 1
        if a.profile_decode_steps and steps_decode == a.profile_decode_steps:
            torch.cuda.synchronize()
            torch.cuda.profiler.stop()
    s2.record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    prefill_ms, decode_ms = s0.elapsed_time(s1), s1.elapsed_time(s2)
    gen = len(prompts) * a.output_tokens
    st = eng.get_stats()
    print(json.dumps({
        "model": a.model_preset, "requests": len(prompts), "prompt_tokens": sum(len(p) for p in prompts),
        "output_tokens": gen, "kv_cache_dtype": a.kv_cache_dtype, "cuda_graph": a.cuda_graph,
        "speculative": a.speculative, "long_context": a.long_context,
        "prefill_ms": prefill_ms, "prefill_tokens_per_s": st["prefill_tokens"] / (prefill_ms * 1e-3),
        "cached_prefix_tokens": st["cached_prefix_tokens"],
        "decode_ms": decode_ms, "decode_steps": steps_decode,
        "decode_ms_per_step": decode_ms / max(1, steps_decode),
        "decode_tokens_per_s": (gen - first) / (decode_ms * 1e-3) if decode_ms > 0 else 0.0,
        "end_to_end_tokens_per_s": gen / ((prefill_ms + decode_ms) * 1e-3),
        # the figure the reference arm (baseline/run_reference_extras.py decode) reports: output tokens over the whole call
        "generation_output_tokens_per_s": gen / ((prefill_ms + decode_ms) * 1e-3), "clocks": clocks,
        "spec_acceptance": st.get("speculative", {}).get("acceptance_rate"),
        "graph_replays": st.get("graph_replays"), "kv_blocks": blocks,
        # who waits for whom with the one-step-late read-back: launches whose result was already there when the host
        # came for it (the host is the limit) against those the host had to wait for (the GPU is), and that wait
        "host_found_result_ready": st.get("inflight_ready", 0), "host_waited_for_gpu": st.get("inflight_waited", 0),
        "host_wait_ms_per_decode_step": 1e3 * st.get("inflight_wait_s", 0.0) / max(1, steps_decode)}))


if __name__ == "__main__":
    main()
