#!/usr/bin/env python
"""Memory profile of one training step: static estimate, per-phase peaks, per-layer peaks, optimizer bytes
(the reference's scripts/profile_memory.py:22-28 flags)."""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

from b200fw.train import TrainConfig, TrainEngine  # noqa: E402


def main():
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--model-preset", default="tiny128")
    ap.add_argument("--model-path", default="")
    ap.add_argument("--batch-size", type=int, default=4)
    ap.add_argument("--seq-len", type=int, default=512)
    ap.add_argument("--lora-rank", type=int, default=0)
    ap.add_argument("--zero-stage", type=int, default=1)
    ap.add_argument("--grad-ckpt", action="store_true")
    ap.add_argument("--output", default="memory_report.json")
    a = ap.parse_args()
    cuda = torch.cuda.is_available()
    cfg = TrainConfig(model_path=a.model_path, model_preset=None if a.model_path else a.model_preset, lora_rank=a.lora_rank,
                      zero_stage=a.zero_stage, use_gradient_checkpoint=a.grad_ckpt, gradient_accumulation_steps=1,
                      grpo_beta=0.0, max_seq_len=a.seq_len, amp_dtype="bf16" if cuda else "fp32", use_amp=cuda)
    eng = TrainEngine(cfg).initialize()
    prof = eng.memory_profiler
    prof.attach_layer_hooks(eng.model)
    ids = torch.randint(0, eng.model_config.vocab_size, (a.batch_size, a.seq_len))
    labels = ids.clone()
    prof.reset_peak()
    eng.sft_step_tensors(ids, labels)
    prof.mark_phase("step")
    rep = eng.generate_memory_report(a.batch_size * a.seq_len)
    rep.save(a.output)
    print(rep.to_text())


if __name__ == "__main__":
    main()
