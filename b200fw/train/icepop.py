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

    def filter_divergent_responses(self, train_log_probs: torch.Tensor, infer_log_probs: torch.Tensor,
                                   advantages: torch.Tensor) -> Tuple[torch.Tensor, Dict[str, float]]:
        gap = (train_log_probs.float() - infer_log_probs.float().to(train_log_probs.device)).abs()
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
        diag = {
            "icepop_masked_ratio": k / max(n, 1),
            "icepop_mean_divergence": gap.mean().item() if n else 0.0,
            "icepop_max_divergence": gap.max().item() if n else 0.0,
            "icepop_num_masked": k,
            "icepop_threshold": self.config.divergence_threshold,
        }
        return out, diag
