#!/usr/bin/env python
"""Colocate training entry point (SFT or GRPO), one process per GPU:

    torchrun --nproc-per-node 8 --master-addr 127.0.0.1 scripts/run_colocate.py --config configs/training/sft.yaml

Same CLI as the reference (scripts/run_colocate.py:31-68): flags override YAML, YAML overrides defaults.
"""
import argparse
import asyncio
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from b200fw.config import apply_determinism, build_colocate_config, load_yaml_config, validate_parallel_config  # noqa: E402
from b200fw.obs import setup_logger  # noqa: E402
from b200fw.orch import ColocateOrchestrator  # noqa: E402


def parse_args(argv=None):
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--config", type=str, default=None)
    ap.add_argument("--model", "--model-path", dest="model_path", type=str, default=None, help="HF model directory")
    ap.add_argument("--model-preset", type=str, default=None, help="random-init architecture (e.g. qwen3-0.6b)")
    ap.add_argument("--tp-size", type=int, default=None)
    ap.add_argument("--dp-size", type=int, default=None)
    ap.add_argument("--pp-size", type=int, default=None)
    ap.add_argument("--iterations", type=int, default=None)
    ap.add_argument("--batch-size", type=int, default=None)
    ap.add_argument("--num-samples", type=int, default=None)
    ap.add_argument("--training-mode", choices=["grpo", "sft"], default=None)
    ap.add_argument("--inference-backend", choices=["vllm", "custom", "native", "mock"], default=None)
    ap.add_argument("--vllm-url", type=str, default=None)
    ap.add_argument("--lr", type=float, default=None)
    ap.add_argument("--lora-rank", type=int, default=None)
    ap.add_argument("--max-tokens", type=int, default=None)
    ap.add_argument("--zero-stage", type=int, default=None)
    ap.add_argument("--resume-from", type=str, default=None)
    ap.add_argument("--output-dir", type=str, default=None)
    ap.add_argument("--synthetic", action="store_true", default=None, help="seeded random-token data + rule reward")
    ap.add_argument("--no-synthetic", dest="synthetic", action="store_false",
                    help="read data.dataset_name (a local JSON / JSONL file or save_to_disk directory) even if the YAML says synthetic")
    ap.add_argument("--log-file", type=str, default=None)
    return ap.parse_args(argv)


def main(argv=None):
    a = parse_args(argv)
    rank = int(os.environ.get("RANK", "0"))
    setup_logger(log_file=a.log_file, rank=rank if a.log_file else None)
    ycfg = load_yaml_config(a.config)
    cfg, unknown = build_colocate_config(ycfg, {
        "model_path": a.model_path, "model_preset": a.model_preset, "tp_size": a.tp_size, "dp_size": a.dp_size,
        "pp_size": a.pp_size, "total_iterations": a.iterations, "batch_size": a.batch_size,
        "num_samples_per_prompt": a.num_samples, "training_mode": a.training_mode,
        "inference_backend": a.inference_backend, "vllm_url": a.vllm_url, "learning_rate": a.lr,
        "lora_rank": a.lora_rank, "max_tokens": a.max_tokens, "zero_stage": a.zero_stage,
        "resume_from": a.resume_from, "output_dir": a.output_dir, "synthetic_data": a.synthetic})
    if unknown and rank == 0:
        print(f"[config] keys not used by this framework: {unknown}", file=sys.stderr)
    validate_parallel_config(cfg)
    apply_determinism(cfg.deterministic, cfg.seed)        # before the first CUDA call: the GEMM reads its switch once

    async def go():
        orch = ColocateOrchestrator(cfg)
        await orch.initialize()
        # SIGTERM (a scheduler reclaiming the node) and the first Ctrl-C end the run at the next iteration boundary
        # with a checkpoint to resume from; a second Ctrl-C interrupts as usual
        import signal

        def stop(signum, _frame):
            orch.request_stop()
            signal.signal(signal.SIGINT, signal.default_int_handler)
            print(f"[run_colocate] signal {signum}: stopping after the current iteration", file=sys.stderr, flush=True)
        for sig in (signal.SIGTERM, signal.SIGINT):
            signal.signal(sig, stop)
        await orch.run()
        summary = orch.get_summary()
        await orch.shutdown()
        return summary

    summary = asyncio.run(go())
    if rank == 0:
        print(json.dumps(summary.get("results", summary), indent=2))


if __name__ == "__main__":
    main()
