"""Synthetic rule reward on token ids: 1.0 if the response contains a seed-derived 3-token target
sequence, plus 0.1 if it ends with EOS, else 0.  Optionally (``dense_weight > 0``) a dense shaping term
is added: ``dense_weight`` times the fraction of response tokens whose id is congruent to the prompt
index modulo 7; it keeps the group-normalised advantages non-zero for a random-init policy, whose
chance of hitting the 3-token target is nil.  Needs no tokenizer and no dataset."""
from __future__ import annotations

import random
from typing import List, Sequence


class SyntheticTokenReward:
    def __init__(self, vocab_size: int, seed: int = 0, eos_token_id: int = 2, target_len: int = 3,
                 target_vocab: int = 0, dense_weight: float = 0.0):
        self.vocab_size, self.seed, self.eos, self.target_len = vocab_size, seed, eos_token_id, target_len
        self.dense_weight = dense_weight
        self.target_vocab = target_vocab or vocab_size
        self.total = 0
        self.hits = 0

    def target_for(self, prompt_index: int) -> List[int]:
        rng = random.Random(self.seed * 1000003 + prompt_index)
        return [rng.randrange(3, self.target_vocab) for _ in range(self.target_len)]

    def score(self, response: Sequence[int], prompt_index: int) -> float:
        tgt = self.target_for(prompt_index)
        n = len(tgt)
        found = any(list(response[i:i + n]) == tgt for i in range(0, max(0, len(response) - n + 1)))
        self.total += 1
        self.hits += int(found)
        dense = 0.0
        if self.dense_weight and len(response) > 0:
            want = prompt_index % 7
            dense = self.dense_weight * sum(1 for t in response if t % 7 == want) / len(response)
        return (1.0 if found else 0.0) + (0.1 if len(response) > 0 and response[-1] == self.eos else 0.0) + dense

    def __call__(self, responses: List[List[Sequence[int]]], prompt_indices: Sequence[int]) -> List[List[float]]:
        return [[self.score(r, pi) for r in group] for group, pi in zip(responses, prompt_indices)]

    def get_stats(self):
        return {"total": self.total, "hit_rate": self.hits / self.total if self.total else 0.0}
