"""Learning-rate schedule: linear warm-up (from 1 % of the peak) followed by cosine / linear decay to
``min_lr_ratio`` of the peak, or constant.  Same shape as the reference's LinearLR + Cosine/Linear
SequentialLR (src/engines/train_engine.py:432-480), as a pure function of the step."""
from __future__ import annotations

import math


class LRSchedule:
    def __init__(self, base_lr: float, kind: str = "cosine", warmup_steps: int = 0, total_steps: int = 0,
                 min_lr_ratio: float = 0.1, warmup_start_factor: float = 0.01):
        assert kind in ("cosine", "linear", "constant")
        self.base_lr, self.kind = base_lr, kind
        self.warmup_steps, self.total_steps = max(0, warmup_steps), max(0, total_steps)
        self.min_lr_ratio, self.warmup_start_factor = min_lr_ratio, warmup_start_factor
        self.step_count = 0

    def lr_at(self, step: int) -> float:
        if self.warmup_steps > 0 and step < self.warmup_steps:
            f = self.warmup_start_factor + (1.0 - self.warmup_start_factor) * step / self.warmup_steps
            return self.base_lr * f
        if self.kind == "constant" or self.total_steps <= self.warmup_steps:
            return self.base_lr
        t = min(1.0, (step - self.warmup_steps) / max(1, self.total_steps - self.warmup_steps))
        lo = self.base_lr * self.min_lr_ratio
        if self.kind == "cosine":
            return lo + (self.base_lr - lo) * 0.5 * (1.0 + math.cos(math.pi * t))
        return self.base_lr + (lo - self.base_lr) * t

    def get_last_lr(self):
        return [self.lr_at(self.step_count)]

    def step(self):
        self.step_count += 1

    def state_dict(self):
        return {"step_count": self.step_count}

    def load_state_dict(self, sd):
        self.step_count = int(sd.get("step_count", 0))
