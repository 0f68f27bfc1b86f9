#!/usr/bin/env python
"""GRPO iteration benchmark (colocate): Qwen3-0.6B-architecture policy with random weights, synthetic
prompts (256 tokens) and rule reward, K responses of up to --max-tokens each, clip 0.2, KL 0.01 against a
frozen reference copy, IcePop and C3PO++ on, full weight sync every iteration.  Prints iteration seconds
with the stage breakdown and the weight-sync milliseconds.  One process per GPU (data parallel)."""
import argparse
import asyncio
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

from b200fw.config import ColocateConfig  # noqa: E402
from b200fw.obs.clocks import ClockSampler  # noqa: E402
from b200fw.orch import ColocateOrchestrator  # noqa: E402


def main():
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--model-preset", default="qwen3-0.6b")
    ap.add_argument("--iterations", type=int, default=3)
    ap.add_argument("--prompts", type=int, default=64)
    ap.add_argument("--num-samples", type=int, default=8)
    ap.add_argument("--prompt-len", type=int, default=256)
    ap.add_argument("--max-tokens", type=int, default=512)
    ap.add_argument("--lora-rank", type=int, default=0)
    ap.add_argument("--zero-stage", type=int, default=2)
    ap.add_argument("--no-c3po", action="store_true")
    ap.add_argument("--async-pipeline", action="store_true")
    ap.add_argument("--dense-reward", type=float, default=0.5,
                    help="weight of the dense shaping term of the synthetic reward (0 = the plain rule reward, which a "
                         "random-init policy never earns: every advantage is then zero and the backward carries no signal)")
    ap.add_argument("--output-dir", default="outputs/bench_grpo")
    a = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if torch.cuda.is_available():
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    cfg = ColocateConfig(
        model_preset=a.model_preset, dp_size=world, training_mode="grpo", total_iterations=a.iterations,
        batch_size=a.prompts, num_samples_per_prompt=a.num_samples, max_tokens=a.max_tokens, temperature=0.8,
        top_p=0.95, lora_rank=a.lora_rank, grpo_beta=0.01, grpo_clip_eps=0.2, gradient_accumulation_steps=1,
        zero_stage=a.zero_stage, inference_backend="native", synthetic_data=True, synthetic_prompt_len=a.prompt_len,
        synthetic_reward_dense_weight=a.dense_reward,
        max_seq_len=a.prompt_len + a.max_tokens, max_data_samples=max(1024, a.prompts * (a.iterations + 2)),
        icepop_enabled=True, c3po_plus_enabled=not a.no_c3po, c3po_plus_token_budget=256,
        c3po_plus_target_batch_tokens=16384, swift_sync_enabled=a.lora_rank > 0,
        async_pipeline_enabled=a.async_pipeline, async_pipeline_max_staleness=1, warmup_steps=0,
        checkpoint_save_enabled=False, output_dir=a.output_dir, tensorboard=False, use_radix_cache=True)

    async def go():
        o = ColocateOrchestrator(cfg)
        await o.initialize()
        await o.run()
        s = o.get_summary()
        await o.shutdown()
        return s, o.metrics

    sampler = ClockSampler(int(os.environ.get("LOCAL_RANK", "0")))
    sampler.start()
    s, metrics = asyncio.run(go())
    clocks = sampler.stop()
    if int(os.environ.get("RANK", "0")) == 0:
        steady = metrics[1:] or metrics
        avg = lambda k: sum(m.state_durations.get(k, 0.0) for m in steady) / len(steady)
        print(json.dumps({"metric": "grpo_iteration_s", "value": sum(m.total_time for m in steady) / len(steady),
                          "n_gpus": world, "rollout_s": avg("inferring"), "train_s": avg("training"),
                          "sync_ms": avg("syncing") * 1e3, "reward_s": avg("rewarding"),
                          "tokens_generated_per_iter": steady[-1].tokens_generated, "dense_reward": a.dense_reward,
                          "avg_reward": sum(m.avg_reward for m in steady) / len(steady), "clocks": clocks,
                          "errors": [m.error for m in metrics if m.error], "results": s["results"]}))


if __name__ == "__main__":
    main()
