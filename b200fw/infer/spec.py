"""Speculative decoding with a native draft model.

Roles as in the reference (src/inference/speculative.py:44-533): the draft proposes ``K`` tokens, the
target scores ``K+1`` positions in ONE forward, acceptance is either greedy (longest matching prefix
plus the target's next token) or sampling-aware (accept with ``min(1, p_t/p_d)``, resample the first
rejection from the normalised residual ``max(0, p_t - p_d)``), and a sliding window tracks the
acceptance rate.  Both models run over paged KV caches; the verify pass is a variable-length prefill
chunk of ``K+1`` tokens per sequence, and rejected positions are trimmed from both caches.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass
from typing import Deque, List, Optional, Tuple

import torch


class AcceptanceTracker:
    def __init__(self, window: int = 100):
        self.events: Deque[Tuple[int, int]] = deque(maxlen=window)

    def record(self, accepted: int, proposed: int):
        self.events.append((accepted, proposed))

    @property
    def rate(self) -> float:
        p = sum(e[1] for e in self.events)
        return sum(e[0] for e in self.events) / p if p else 1.0


def verify_greedy(draft_tokens: torch.Tensor, target_logits: torch.Tensor) -> Tuple[int, int]:
    """``draft_tokens [K]``, ``target_logits [K+1, V]`` -> (accepted count, next token)."""
    pred = target_logits.argmax(-1)
    K = draft_tokens.numel()
    match = (pred[:K] == draft_tokens).long()
    n = int(match.cumprod(0).sum())
    return n, int(pred[n])


def verify_sampling(draft_tokens: torch.Tensor, draft_probs: torch.Tensor, target_logits: torch.Tensor,
                    temperature: float, generator: Optional[torch.Generator] = None) -> Tuple[int, int]:
    """Sampling-aware acceptance that preserves the target distribution.  ``draft_probs [K, V]`` are the
    distributions the draft sampled from; returns (accepted count, next token)."""
    K = draft_tokens.numel()
    pt = torch.softmax(target_logits.float() / max(temperature, 1e-6), -1)
    u = torch.rand(K, device=pt.device, generator=generator)
    for i in range(K):
        tok = int(draft_tokens[i])
        ratio = pt[i, tok] / draft_probs[i, tok].clamp(min=1e-20)
        if float(u[i]) < float(ratio.clamp(max=1.0)):
            continue
        resid = (pt[i] - draft_probs[i]).clamp(min=0)
        s = resid.sum()
        resid = resid / s if float(s) > 0 else pt[i]
        return i, int(torch.multinomial(resid, 1, generator=generator))
    return K, int(torch.multinomial(pt[K], 1, generator=generator))


def verify_greedy_batch(draft_tokens: torch.Tensor, target_logits: torch.Tensor):
    """Batched :func:`verify_greedy`: ``draft_tokens [B,K]``, ``target_logits [B,K+1,V]`` ->
    ``(accepted [B], next_token [B])`` as device tensors (no host sync)."""
    pred = target_logits.argmax(-1)
    K = draft_tokens.shape[1]
    n = (pred[:, :K] == draft_tokens).long().cumprod(1).sum(1)
    return n, pred.gather(1, n[:, None]).squeeze(1)


def verify_sampling_batch(draft_tokens: torch.Tensor, draft_probs: torch.Tensor, target_logits: torch.Tensor,
                          temperature: float, generator: Optional[torch.Generator] = None):
    """Batched :func:`verify_sampling` (same acceptance rule, one draw of uniforms per position and one
    residual / bonus draw per sequence).  Returns ``(accepted [B], next_token [B])`` on the device."""
    B, K = draft_tokens.shape
    pt = torch.softmax(target_logits.float() / max(temperature, 1e-6), -1)          # [B,K+1,V]
    idx = draft_tokens[..., None]
    ratio = pt[:, :K].gather(2, idx).squeeze(2) / draft_probs.gather(2, idx).squeeze(2).clamp(min=1e-20)
    u = torch.rand(B, K, device=pt.device, generator=generator)
    n = (u < ratio.clamp(max=1.0)).long().cumprod(1).sum(1)                         # first rejection
    rows = torch.arange(B, device=pt.device)
    p_at = pt[rows, n]                                                              # [B,V]
    d_at = draft_probs[rows, n.clamp(max=K - 1)]
    resid = (p_at - d_at).clamp(min=0)
    ssum = resid.sum(-1, keepdim=True)
    resid = torch.where(ssum > 0, resid / ssum.clamp(min=1e-30), p_at)
    dist = torch.where((n == K)[:, None], p_at, resid)
    return n, torch.multinomial(dist, 1, generator=generator).squeeze(1)


@dataclass
class SpeculativeConfig:
    """The reference's knobs (src/inference/speculative.py:29-41)."""
    enabled: bool = False
    draft_model_path: str = ""
    num_speculative_tokens: int = 5
    temperature: float = 0.0                    # draft sampling temperature (0 = greedy)
    use_batch_draft: bool = True
    use_sampling_verification: bool = False
    verification_temperature: float = 1.0
    verification_top_p: float = 0.9
    min_acceptance_prob: float = 0.1


class SpeculativeDecoder:
    """Drives draft + target runners for a batch of sequences that already finished prefill in both
    caches.  ``target`` / ``draft`` are :class:`ModelRunner` objects with their own block managers."""

    def __init__(self, target, draft, num_tokens: int = 4, window: int = 100,
                 config: Optional[SpeculativeConfig] = None):
        self.config = config or SpeculativeConfig(enabled=True, num_speculative_tokens=num_tokens)
        if config is not None:
            num_tokens = config.num_speculative_tokens
        self.target, self.draft, self.K = target, draft, num_tokens
        self.tracker = AcceptanceTracker(window)
        self.steps = 0
        self.total_proposed = 0
        self.total_accepted = 0
        self._last_sync_count = 0

    @property
    def acceptance_rate(self) -> float:
        return self.tracker.rate

    # ---- the reference's stateless API (src/inference/speculative.py:71-533): one sequence, tensors in and out,
    # no paged caches involved.  The engine uses :meth:`step` instead. --------------------------------------------
    @property
    def is_loaded(self) -> bool:
        return self.draft is not None

    def load_draft_model(self) -> bool:
        """The draft runner is handed to the constructor already built (the engine builds it from
        ``speculative_draft_model_path`` or as a shallow random-init model); reports whether there is one."""
        return self.is_loaded

    def _draft_module(self):
        return getattr(self.draft, "model", self.draft)

    @torch.no_grad()
    def speculate(self, input_ids: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """``input_ids [1, S]`` -> ``(draft_tokens [K], draft_logits [K, V])`` by K full re-forwards of the draft."""
        assert self.is_loaded, "Draft model not loaded"
        ids = input_ids
        toks, logs = [], []
        t = self.config.temperature
        for _ in range(self.K):
            logits = self._draft_module()(ids)[:, -1].float()
            nxt = logits.argmax(-1) if t <= 0 else torch.multinomial(torch.softmax(logits / t, -1), 1).squeeze(-1)
            toks.append(nxt)
            logs.append(logits[0])
            ids = torch.cat([ids, nxt[:, None]], 1)
        return torch.cat(toks), torch.stack(logs)

    def verify(self, input_ids: torch.Tensor, draft_tokens: torch.Tensor, target_logits: torch.Tensor,
               draft_logits: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, int]:
        """``target_logits [1, K+1, V]`` over (last token, draft tokens) -> ``(accepted tokens followed by the
        target's own next token, number of draft tokens accepted)``.  Greedy prefix match, or the sampling-aware
        rule when ``config.use_sampling_verification`` and ``draft_logits`` are given."""
        tl = target_logits[0] if target_logits.dim() == 3 else target_logits
        if self.config.use_sampling_verification and draft_logits is not None:
            temp = self.config.verification_temperature
            dp = torch.softmax(draft_logits.float() / max(temp, 1e-6), -1)
            n, nxt = verify_sampling(draft_tokens, dp, tl, temp)
        else:
            n, nxt = verify_greedy(draft_tokens, tl)
        self._account(n, draft_tokens.numel())
        return torch.cat([draft_tokens[:n], torch.tensor([nxt], dtype=draft_tokens.dtype, device=draft_tokens.device)]), n

    def sync_kv_cache(self, accepted_tokens: torch.Tensor, target_kv_cache=None):
        """Marks how many tokens the caller has to add to the target cache.  With the paged runners nothing is
        left to do: :meth:`step` trims both caches to the accepted history itself."""
        self._last_sync_count = int(accepted_tokens.numel())

    def _account(self, accepted: int, proposed: int):
        self.tracker.record(accepted, proposed)
        self.total_accepted += accepted
        self.total_proposed += proposed

    def get_stats(self) -> dict:
        return {"enabled": self.config.enabled, "loaded": self.is_loaded, "acceptance_rate": self.acceptance_rate,
                "total_proposed": self.total_proposed, "total_accepted": self.total_accepted,
                "num_speculative_tokens": self.K, "history_window_size": len(self.tracker.events),
                "rounds": self.steps}

    def can_step(self, seq_ids: List) -> bool:
        """True when both caches have room for a whole round of every sequence (K draft tokens + the catch-up slot in
        the draft cache, K + 1 verified positions in the target cache).  A round that ran out of blocks half-way would
        leave the two caches at different lengths; the engine asks first and decodes normally when the answer is no."""
        for runner, extra in ((self.draft, self.K + 1), (self.target, self.K + 1)):
            mgr, need = runner.mgr, 0
            for s in seq_ids:
                table = mgr.tables.get(s)
                if table is None:
                    return False
                need += max(0, mgr.blocks_needed(table.num_tokens + extra) - table.num_blocks)
            if need > mgr.pool.num_free_blocks:
                return False
        return True

    def _draft_propose(self, seq_ids: List, last_tokens: List[int], temperature: float,
                       generator=None) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        """K draft decode steps for all sequences.  Returns tokens ``[B, K]`` and, when sampling, the
        draft distributions ``[B, K, V]``."""
        dev = self.draft.device
        B = len(seq_ids)
        cur = torch.tensor(last_tokens, dtype=torch.long, device=dev)
        toks, probs = [], []
        for _ in range(self.K):
            for s in seq_ids:
                if not self.draft.mgr.append_token(s):
                    raise RuntimeError("draft KV cache exhausted")
            ctx = self.draft.prepare_decode(seq_ids)
            logits = self.draft.forward(cur, ctx)
            if temperature <= 0:
                cur = logits.argmax(-1)
            else:
                p = torch.softmax(logits.float() / temperature, -1)
                cur = torch.multinomial(p, 1, generator=generator).squeeze(-1)
                probs.append(p)
            toks.append(cur)
        return torch.stack(toks, 1), (torch.stack(probs, 1) if probs else None)

    def step(self, seq_ids: List, last_tokens: List[int], temperature: float = 0.0,
             generator: Optional[torch.Generator] = None) -> List[List[int]]:
        """One speculative round.  ``last_tokens[i]`` is the newest token of sequence ``i`` that is not
        in either cache yet.  Returns the new tokens per sequence (1 .. K+1 each) and leaves both caches
        holding exactly the accepted history (without the final returned token)."""
        K = self.K
        tgt, dr = self.target, self.draft
        base = [tgt.mgr.get_seq_token_count(s) for s in seq_ids]
        d_tokens, d_probs = self._draft_propose(seq_ids, last_tokens, temperature, generator)
        # target verifies [last, d_0 .. d_{K-1}] in one variable-length chunk per sequence
        for s, b in zip(seq_ids, base):
            if not tgt.mgr.ensure_capacity(s, b + K + 1):
                raise RuntimeError("target KV cache exhausted")
            tgt.mgr.set_num_tokens(s, b + K + 1)
        ctx = tgt.prepare_prefill(seq_ids, base, [K + 1] * len(seq_ids))
        ids = torch.cat([torch.tensor(last_tokens, dtype=torch.long, device=tgt.device)[:, None], d_tokens], 1)
        logits = tgt.forward(ids.reshape(-1), ctx, all_rows=True).reshape(len(seq_ids), K + 1, -1)
        out: List[List[int]] = []
        catch_up: List[int] = []
        if temperature <= 0:
            n_dev, nxt_dev = verify_greedy_batch(d_tokens, logits)
        else:
            n_dev, nxt_dev = verify_sampling_batch(d_tokens, d_probs, logits, temperature, generator)
        # the only host sync of the round: accepted counts, next tokens and the drafts in one copy
        packed = torch.cat([n_dev[:, None], nxt_dev[:, None], d_tokens], 1).tolist()
        for i, s in enumerate(seq_ids):
            n, nxt = packed[i][0], packed[i][1]
            self._account(n, K)
            out.append(packed[i][2:2 + n] + [nxt])
            # both caches must end up holding history + last + the n accepted drafts; the returned
            # final token is the next round's `last` and is not stored yet
            tgt.mgr.trim(s, base[i] + 1 + n)
            if n < K:
                dr.mgr.trim(s, base[i] + 1 + n)
            else:
                catch_up.append(i)      # the draft produced d_{K-1} but never consumed it
        if catch_up:
            ids_c = [seq_ids[i] for i in catch_up]
            for s in ids_c:
                if not dr.mgr.append_token(s):
                    raise RuntimeError("draft KV cache exhausted")
            ctx_c = dr.prepare_decode(ids_c)
            dr.forward(d_tokens[catch_up, K - 1].contiguous(), ctx_c)
        self.steps += 1
        return out
