#!/usr/bin/env python
"""Memory profile of one training step: static estimate, per-phase peaks, per-layer peaks, optimizer bytes
(the reference's scripts/profile_memory.py:22-28 flags)."""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

from b200fw.train import TrainConfig, TrainEngine  # noqa: E402


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--config", default=None, help="training YAML (model / runtime / training / lora sections)")
    ap.add_argument("--model-preset", default=None)
    ap.add_argument("--model-path", default="")
    ap.add_argument("--batch-size", type=int, default=None)
    ap.add_argument("--seq-len", type=int, default=None)
    ap.add_argument("--lora-rank", type=int, default=None)
    ap.add_argument("--zero-stage", type=int, default=None)
    ap.add_argument("--grad-ckpt", action="store_true", default=None)
    ap.add_argument("--device", default=None, help="cuda:N or cpu (default: cuda:0 when there is one)")
    ap.add_argument("--skip-backward", action="store_true", help="profile the forward pass only")
    ap.add_argument("--output", default=None, help="report path (default: outputs/memory_report.json)")
    a = ap.parse_args(argv)
    from b200fw.config import build_colocate_config, load_yaml_config
    cc, _ = build_colocate_config(load_yaml_config(a.config), {
        "model_path": a.model_path or None, "model_preset": a.model_preset, "batch_size": a.batch_size,
        "max_seq_len": a.seq_len, "lora_rank": a.lora_rank, "zero_stage": a.zero_stage,
        "use_gradient_checkpoint": a.grad_ckpt})
    if a.config is None and not a.model_path and a.model_preset is None:
        cc.model_preset = "tiny128"
    if a.config is None:
        cc.batch_size = a.batch_size or 4
        cc.max_seq_len = a.seq_len or 512
        cc.lora_rank = a.lora_rank or 0
    cuda = torch.cuda.is_available() and (a.device or "cuda").startswith("cuda")
    if cuda and a.device and ":" in a.device:
        torch.cuda.set_device(int(a.device.split(":")[1]))
    # one process: the parallel sizes of the YAML enter the static estimate, not the run
    cfg = TrainConfig(model_path="" if cc.model_preset else cc.model_path, model_preset=cc.model_preset,
                      lora_rank=cc.lora_rank, lora_alpha=cc.lora_alpha, zero_stage=min(cc.zero_stage, 1),
                      use_gradient_checkpoint=cc.use_gradient_checkpoint, gradient_accumulation_steps=1, grpo_beta=0.0,
                      max_seq_len=cc.max_seq_len, amp_dtype="bf16" if cuda else "fp32", use_amp=cuda,
                      backend=None if cuda else "gloo")
    eng = TrainEngine(cfg).initialize()
    prof = eng.memory_profiler
    prof.attach_layer_hooks(eng.model)
    B, S = max(1, cc.batch_size), cc.max_seq_len
    ids = torch.randint(0, eng.model_config.vocab_size, (B, S))
    labels = ids.clone()
    prof.reset_peak()
    if a.skip_backward:
        eng.eval_sft_loss(ids[:, : S // 2].tolist(), ids[:, S // 2:].tolist())
        prof.mark_phase("forward")
    else:
        eng.sft_step_tensors(ids, labels)
        prof.mark_phase("step")
    rep = eng.generate_memory_report(B * S)
    out = a.output or os.path.join("outputs", "memory_report.json")
    os.makedirs(os.path.dirname(os.path.abspath(out)), exist_ok=True)
    rep.save(out)
    print(rep.to_text())
    return rep


if __name__ == "__main__":
    main()
