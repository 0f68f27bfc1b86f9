"""C3PO++: split long rollouts into token-budget chunks and bin-pack them into balanced sub-batches.

Same contract as the reference scheduler (src/engines/c3po_plus.py:58-305): chunk ``k`` of a response
is trained with ``prompt + earlier response tokens`` as its prompt; chunks are packed first-fit-
decreasing by ``prompt + prefix + chunk`` length into bins of ``target_batch_tokens``; each bin becomes
``grpo_step`` keyword arguments with one response per (extended) prompt and advantages computed on
the *whole* responses beforehand, so splitting does not change the group statistics.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple


@dataclass
class C3POConfig:
    enabled: bool = False
    token_budget: int = 1024
    target_batch_tokens: int = 4096
    packing_strategy: str = "ffd"


@dataclass
class ResponseChunk:
    prompt_tokens: List[int]
    response_tokens: List[int]
    response_prefix: List[int]
    reward: float
    source_idx: Tuple[int, int]
    advantage: float = 0.0
    infer_logprob: Optional[float] = None       # mean rollout log-prob of this chunk's tokens (IcePop), when known

    @property
    def length(self) -> int:
        return len(self.prompt_tokens) + len(self.response_prefix) + len(self.response_tokens)


class C3POPlusScheduler:
    def __init__(self, config: C3POConfig):
        self.config = config
        self.last_stats: Dict[str, float] = {}

    def split(self, prompts_tokens, responses_group, rewards_group, advantages_group=None,
              token_logprobs_group=None) -> List[ResponseChunk]:
        """``token_logprobs_group[b][k]``: the rollout engine's per-token log-probs of response ``k`` of prompt ``b``
        (optional); each chunk then carries the mean over its own tokens, so IcePop can compare it with the
        trainer's without an extra inference-mode forward."""
        budget = max(1, self.config.token_budget)
        chunks: List[ResponseChunk] = []
        for b, (prompt, responses, rewards) in enumerate(zip(prompts_tokens, responses_group, rewards_group)):
            for k, (resp, rew) in enumerate(zip(responses, rewards)):
                adv = advantages_group[b][k] if advantages_group is not None else 0.0
                tlp = token_logprobs_group[b][k] if token_logprobs_group is not None else None
                starts = range(0, max(len(resp), 1), budget)
                for s in starts:
                    lp = None
                    if tlp is not None and len(tlp) >= min(len(resp), s + budget) and len(resp) > s:
                        piece = tlp[s:s + budget]
                        lp = sum(piece) / len(piece)
                    chunks.append(ResponseChunk(prompt, resp[s:s + budget], resp[:s], rew, (b, k), adv, lp))
        return chunks

    def pack(self, chunks: List[ResponseChunk]) -> List[List[ResponseChunk]]:
        cap = self.config.target_batch_tokens
        if self.config.packing_strategy != "ffd":
            raise ValueError(f"unknown packing strategy {self.config.packing_strategy!r}")
        bins: List[List[ResponseChunk]] = []
        load: List[int] = []
        for c in sorted(chunks, key=lambda c: c.length, reverse=True):
            slot = next((i for i, l in enumerate(load) if l + c.length <= cap), None) if c.length <= cap else None
            if slot is None:
                bins.append([c])
                load.append(c.length)
            else:
                bins[slot].append(c)
                load[slot] += c.length
        self.last_stats = {"chunks": len(chunks), "bins": len(bins), "max_bin_tokens": max(load, default=0),
                           "mean_fill": (sum(load) / (len(load) * cap)) if load else 0.0}
        return bins

    @staticmethod
    def to_grpo_kwargs(bin_chunks: List[ResponseChunk]) -> Dict:
        kw = {
            "prompts_tokens": [c.prompt_tokens + c.response_prefix for c in bin_chunks],
            "responses_group": [[c.response_tokens] for c in bin_chunks],
            "rewards_group": [[c.reward] for c in bin_chunks],
            "precomputed_advantages": [[c.advantage] for c in bin_chunks],
        }
        if bin_chunks and all(c.infer_logprob is not None for c in bin_chunks):
            import torch
            kw["infer_log_probs"] = torch.tensor([c.infer_logprob for c in bin_chunks], dtype=torch.float32)
        return kw

    def split_and_pack(self, prompts_tokens: List[List[int]], responses_group: List[List[List[int]]],
                       rewards_group: List[List[float]],
                       advantages_group: Optional[List[List[float]]] = None,
                       token_logprobs_group=None) -> List[Dict]:
        chunks = self.split(prompts_tokens, responses_group, rewards_group, advantages_group, token_logprobs_group)
        return [self.to_grpo_kwargs(b) for b in self.pack(chunks)]
