#!/usr/bin/env python
"""Disaggregated GRPO: trainer ranks and rollout ranks in one world.

    torchrun --nproc-per-node 8 --master-addr 127.0.0.1 scripts/run_disaggregated.py \
        --model-preset qwen3-0.6b --num-train-gpus 4 --num-infer-gpus 4

CLI after the reference's (scripts/run_disaggregated.py:26-56); Ray is replaced by rank groups.
"""
import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

from b200fw.dist.context import ParallelContext  # noqa: E402
from b200fw.infer import InferenceConfig, InferenceEngine  # noqa: E402
from b200fw.model import PRESETS, ParallelTransformerModel, read_hf_config  # noqa: E402
from b200fw.orch import DisaggConfig, DisaggOrchestrator  # noqa: E402
from b200fw.train import TrainConfig, TrainEngine  # noqa: E402


def parse_args(argv=None):
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--model", "--model-path", dest="model_path", default="", help="HF model directory")
    ap.add_argument("--model-preset", default=None)
    ap.add_argument("--num-train-gpus", "--train-tp", dest="num_train_gpus", type=int, default=4,
                    help="ranks in the trainer group (data parallel + ZeRO; the reference's --train-tp sized its "
                         "trainer actor the same way)")
    ap.add_argument("--num-infer-gpus", "--infer-tp", dest="num_infer_gpus", type=int, default=4,
                    help="ranks running rollout engines (one engine per rank)")
    ap.add_argument("--iterations", type=int, default=4)
    ap.add_argument("--batch-size", type=int, default=64)
    ap.add_argument("--num-samples", type=int, default=8)
    ap.add_argument("--prompt-len", type=int, default=256)
    ap.add_argument("--max-tokens", type=int, default=512)
    ap.add_argument("--zero-stage", type=int, default=2)
    ap.add_argument("--lora-rank", type=int, default=0)
    ap.add_argument("--lr", type=float, default=1e-5)
    ap.add_argument("--mode", choices=["pipeline", "sequential"], default="pipeline")
    ap.add_argument("--no-overlap", action="store_true", help="same as --mode sequential")
    ap.add_argument("--transfer-backend", "--weight-backend", dest="transfer_backend",
                    choices=["nccl", "peer_write", "ray"], default="nccl",
                    help="'ray' (object store) is not available in a torchrun world and falls back to nccl")
    ap.add_argument("--kv-cache-dtype", choices=["fp16", "fp8"], default="fp16")
    ap.add_argument("--backend", default=None)
    ap.add_argument("--log-file", default=None)
    ap.add_argument("--dataset", default=None, help="local JSON / JSONL file or save_to_disk directory with question / "
                                                    "answer fields (default: seeded random-token prompts + token-rule reward)")
    ap.add_argument("--prompt-template", default="qwen3_math")
    return ap.parse_args(argv)


def main(argv=None):
    a = parse_args(argv)
    if a.no_overlap:
        a.mode = "sequential"
    if a.transfer_backend == "ray":
        a.transfer_backend = "nccl"
    if a.log_file:
        from b200fw.obs import setup_logger
        setup_logger("b200fw", log_file=a.log_file)
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    cuda = torch.cuda.is_available()
    if cuda:
        torch.cuda.set_device(local)
    backend = a.backend or ("nccl" if cuda else "gloo")
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29500")
    dist.init_process_group(backend, rank=rank, world_size=world)
    mc = PRESETS[a.model_preset] if a.model_preset else read_hf_config(a.model_path)
    cfg = DisaggConfig(a.model_path, a.model_preset, a.num_train_gpus, a.num_infer_gpus, a.zero_stage, a.iterations,
                       a.batch_size, a.num_samples, a.prompt_len, a.max_tokens, learning_rate=a.lr, lora_rank=a.lora_rank, mode=a.mode,
                       transfer_backend=a.transfer_backend, kv_cache_dtype=a.kv_cache_dtype)

    def make_trainer(group, n, r):
        ctx = ParallelContext(1, n, 1, r, n, local, backend)
        ctx.dp_group, ctx.dp_ranks = (group if n > 1 else None), list(range(n))
        ParallelContext._instance = ctx
        tc = TrainConfig(model_path=a.model_path, model_preset=a.model_preset, dp_size=n, lora_rank=a.lora_rank,
                         zero_stage=a.zero_stage, gradient_accumulation_steps=1, grpo_beta=cfg.grpo_beta, learning_rate=a.lr,
                         max_seq_len=a.prompt_len + a.max_tokens, warmup_steps=0,
                         amp_dtype="bf16" if cuda else "fp32", use_amp=cuda)
        return TrainEngine(tc).initialize(ctx)

    def make_engine(i):
        dev = torch.device("cuda", local) if cuda else torch.device("cpu")
        model = ParallelTransformerModel(mc, dtype=torch.bfloat16 if cuda else torch.float32, device=dev)
        model.init_weights(0)
        for p in model.parameters():
            p.requires_grad_(False)
        seqs = -(-a.batch_size // max(1, a.num_infer_gpus)) * a.num_samples
        blocks = cfg.kv_num_blocks or int(seqs * (-(-(a.prompt_len + a.max_tokens) // 16) + 1) * 1.1) + 64
        ic = InferenceConfig.from_model_config(mc, num_blocks=blocks, inference_mode="kv_cache",
                                               kv_cache_dtype=a.kv_cache_dtype, max_num_batched_tokens=8192,
                                               max_prefill_tokens=4096, seed=i)
        return InferenceEngine(ic, model).initialize()

    data = None
    if a.dataset:
        from b200fw.data import GSM8KDataPipeline
        data = GSM8KDataPipeline(tokenizer_name=a.model_path or None, dataset_name=a.dataset,
                                 prompt_template=a.prompt_template, max_prompt_tokens=a.prompt_len)
    orch = DisaggOrchestrator(cfg, make_trainer, make_engine, data=data).initialize()
    orch.run()
    summaries = [None] * world
    dist.all_gather_object(summaries, orch.get_summary())
    if rank == 0:
        print(json.dumps({"trainer": summaries[0], "rollout": summaries[-1]}, indent=2))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
