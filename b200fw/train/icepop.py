"""IcePop: drop responses whose sequence log-prob under the trainer diverges from the rollout engine's.

Behaviour of the reference filter (src/engines/icepop.py:48-122): a response is anomalous when
``|train_lp - infer_lp| > divergence_threshold``; at most ``max_mask_ratio`` of the responses are
masked, the most divergent first; masked responses get advantage 0 and so contribute no gradient.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Tuple

import torch


@dataclass
class IcePopConfig:
    enabled: bool = False
    divergence_threshold: float = 0.5
    max_mask_ratio: float = 0.5
    log_diagnostics: bool = True


class IcePopFilter:
    def __init__(self, config: IcePopConfig):
        self.config = config
        self.total_seen = 0
        self.total_masked = 0
        self.last_non_finite = 0

    def filter_divergent_responses(self, train_log_probs: torch.Tensor, infer_log_probs: torch.Tensor,
                                   advantages: torch.Tensor) -> Tuple[torch.Tensor, Dict[str, float]]:
        gap = (train_log_probs.float() - infer_log_probs.float().to(train_log_probs.device)).abs()
        # a log-prob that is not a number on either side is the strongest possible disagreement, not "no disagreement"
        # (a comparison with NaN is false, which would let such a response through with its advantage intact)
        finite = torch.isfinite(gap)
        gap = torch.where(finite, gap, torch.full_like(gap, float("inf")))
        n = advantages.shape[0]
        cap = int(n * self.config.max_mask_ratio)
        over = gap > self.config.divergence_threshold
        # rank the anomalous ones by divergence and keep at most `cap` of them
        score = torch.where(over, gap, torch.full_like(gap, -1.0))
        k = min(cap, int(over.sum().item()))
        drop = torch.zeros_like(over)
        if k > 0:
            drop[score.topk(k).indices] = True
        out = torch.where(drop, torch.zeros_like(advantages), advantages)
        self.total_seen += n
        self.total_masked += k
        self.last_non_finite = int((~finite).sum().item())      # kept off the diagnostics dict: its key set is the reference's
        diag = {
            "icepop_masked_ratio": k / max(n, 1),
            "icepop_mean_divergence": gap[finite].mean().item() if bool(finite.any()) else 0.0,
            "icepop_max_divergence": gap[finite].max().item() if bool(finite.any()) else 0.0,
            "icepop_num_masked": k,
            "icepop_threshold": self.config.divergence_threshold,
        }
        return out, diag
