"""Continuous-batching scheduler (policy of src/inference/scheduler.py:141-378).

Decode first: every running sequence gets one token of budget; if that alone exceeds the token or
sequence limits, the most recently arrived running sequence is preempted (its progress is reset and it
goes back to the *head* of the waiting queue).  The remaining budget (capped by ``max_prefill_tokens``)
admits waiting requests first come first served, at most one chunk each; the chunk adapts to load
(halved with more than 3 running sequences, doubled when idle); the first request may take whatever
budget is left even if that is less than a chunk.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from enum import Enum
from typing import Dict, List, Optional


class RequestState(Enum):
    WAITING = "waiting"
    RUNNING = "running"
    FINISHED = "finished"
    PREEMPTED = "preempted"


@dataclass
class Request:
    request_id: str
    prompt_tokens: List[int]
    max_tokens: int = 512
    temperature: float = 0.7
    top_p: float = 0.9
    state: RequestState = RequestState.WAITING
    output_tokens: List[int] = field(default_factory=list)
    output_logprobs: List[float] = field(default_factory=list)
    num_computed_tokens: int = 0
    arrival_time: float = field(default_factory=time.time)
    eos_token_id: Optional[int] = 2
    num_cached_tokens: int = 0          # prompt tokens served from the prefix cache
    preemptions: int = 0

    @property
    def num_prompt_tokens(self) -> int:
        return len(self.prompt_tokens)

    @property
    def num_generated_tokens(self) -> int:
        return len(self.output_tokens)

    @property
    def total_tokens(self) -> int:
        return self.num_prompt_tokens + self.num_generated_tokens

    @property
    def is_prefill_complete(self) -> bool:
        return self.num_computed_tokens >= self.num_prompt_tokens

    @property
    def remaining_prefill_tokens(self) -> int:
        return max(0, self.num_prompt_tokens - self.num_computed_tokens)

    @property
    def is_finished(self) -> bool:
        if self.num_generated_tokens >= self.max_tokens:
            return True
        return bool(self.output_tokens) and self.eos_token_id is not None and self.output_tokens[-1] == self.eos_token_id


@dataclass
class SchedulerOutput:
    prefill_requests: List[Request] = field(default_factory=list)
    decode_requests: List[Request] = field(default_factory=list)
    preempted_requests: List[Request] = field(default_factory=list)
    chunk_size: int = 512
    prefill_tokens: Dict[str, int] = field(default_factory=dict)    # request id -> tokens scheduled now

    @property
    def num_prefill_tokens(self) -> int:
        if self.prefill_tokens:
            return sum(self.prefill_tokens.values())
        return sum(min(r.remaining_prefill_tokens, self.chunk_size) for r in self.prefill_requests)

    @property
    def num_decode_tokens(self) -> int:
        return len(self.decode_requests)

    @property
    def total_tokens(self) -> int:
        return self.num_prefill_tokens + self.num_decode_tokens

    @property
    def is_empty(self) -> bool:
        return not self.prefill_requests and not self.decode_requests


class ContinuousBatchingScheduler:
    def __init__(self, max_num_batched_tokens: int = 2048, max_num_sequences: int = 256,
                 max_prefill_tokens: int = 1024, enable_chunked_prefill: bool = True, chunk_size: int = 512,
                 enable_adaptive_chunking: bool = True):
        self.max_num_batched_tokens, self.max_num_sequences = max_num_batched_tokens, max_num_sequences
        self.max_prefill_tokens, self.enable_chunked_prefill = max_prefill_tokens, enable_chunked_prefill
        self.chunk_size, self.enable_adaptive_chunking = chunk_size, enable_adaptive_chunking
        self.waiting_queue: List[Request] = []
        self.running_queue: List[Request] = []
        self.total_scheduled = self.total_preempted = self.total_finished = 0
        # Optional hook ``defer(request) -> bool``: a not-yet-started request for which it returns True
        # is skipped this step (the engine uses it to hold back requests whose prompt prefix is being
        # prefilled by another request right now, so that they can share its blocks one step later).
        self.defer = None

    def add_request(self, request: Request):
        request.state = RequestState.WAITING
        self.waiting_queue.append(request)

    def _adaptive_chunk(self) -> int:
        if not self.enable_adaptive_chunking:
            return self.chunk_size
        n = len(self.running_queue)
        if n > 3:
            return max(self.chunk_size // 2, 128)
        if n == 0:
            return min(self.chunk_size * 2, 2048)
        return self.chunk_size

    def requeue(self, request: Request):
        """Put a request whose scheduled work could not start (no KV blocks right now) back at the head of the waiting
        queue with its progress untouched; it is offered again at the next step."""
        if request in self.running_queue:
            self.running_queue.remove(request)
        if request in self.waiting_queue:
            self.waiting_queue.remove(request)
        request.state = RequestState.WAITING
        self.waiting_queue.insert(0, request)

    def preempt(self, victim: Request) -> Request:
        """Evict ``victim`` (running, or waiting with part of its prompt computed): its progress is reset, it returns
        to the head of the waiting queue and is recomputed later.  The caller frees its KV blocks."""
        if victim in self.running_queue:
            self.running_queue.remove(victim)
        if victim in self.waiting_queue:
            self.waiting_queue.remove(victim)
        victim.num_computed_tokens = 0
        victim.output_tokens.clear()
        victim.output_logprobs.clear()
        victim.preemptions += 1
        victim.state = RequestState.WAITING
        self.waiting_queue.insert(0, victim)
        self.total_preempted += 1
        return victim

    def preempt_one(self) -> Optional[Request]:
        if not self.running_queue:
            return None
        i = max(range(len(self.running_queue)), key=lambda j: self.running_queue[j].arrival_time)
        victim = self.running_queue.pop(i)
        victim.num_computed_tokens = 0
        victim.output_tokens.clear()
        victim.output_logprobs.clear()
        victim.preemptions += 1
        victim.state = RequestState.WAITING
        self.waiting_queue.insert(0, victim)
        self.total_preempted += 1
        return victim

    def schedule(self) -> SchedulerOutput:
        out = SchedulerOutput(chunk_size=self.chunk_size)
        while len(self.running_queue) > min(self.max_num_batched_tokens, self.max_num_sequences):
            v = self.preempt_one()
            if v is None:
                break
            out.preempted_requests.append(v)
        out.decode_requests = list(self.running_queue)
        budget = min(self.max_num_batched_tokens - len(self.running_queue), self.max_prefill_tokens)
        slots = self.max_num_sequences - len(self.running_queue)
        if budget > 0 and slots > 0 and self.waiting_queue:
            chunk = self._adaptive_chunk()
            out.chunk_size = chunk
            done_idx = []
            for r in [w for w in self.waiting_queue if w.is_prefill_complete and w.num_prompt_tokens > 0]:
                self.promote_if_prefilled(r)
            for i, r in enumerate(self.waiting_queue):
                if len(out.prefill_requests) >= slots:
                    break
                if self.defer is not None and r.num_computed_tokens == 0 and self.defer(r):
                    continue
                want = r.remaining_prefill_tokens
                if self.enable_chunked_prefill:
                    want = min(want, chunk)
                if want > budget:
                    if out.prefill_requests:
                        break
                    want = budget               # the first request takes what is left
                if want <= 0:
                    break
                budget -= want
                out.prefill_requests.append(r)
                out.prefill_tokens[r.request_id] = want
                if r.num_computed_tokens + want >= r.num_prompt_tokens:
                    done_idx.append(i)
            for i in reversed(done_idx):
                r = self.waiting_queue.pop(i)
                r.state = RequestState.RUNNING
                self.running_queue.append(r)
        self.total_scheduled += 1
        return out

    def promote_if_prefilled(self, request: Request):
        """A request whose prompt is fully computed (e.g. a cached prefix made its first chunk the last
        one) moves from the waiting to the running queue."""
        if request.is_prefill_complete and request in self.waiting_queue:
            self.waiting_queue.remove(request)
            request.state = RequestState.RUNNING
            self.running_queue.append(request)

    def update_request_progress(self, request_id: str, num_new_tokens: int):
        for q in (self.waiting_queue, self.running_queue):
            for r in q:
                if r.request_id == request_id:
                    r.num_computed_tokens += num_new_tokens
                    return

    def finish_request(self, request_id: str):
        for q in (self.running_queue, self.waiting_queue):
            for i, r in enumerate(q):
                if r.request_id == request_id:
                    q.pop(i)
                    r.state = RequestState.FINISHED
                    self.total_finished += 1
                    return

    def abort_all(self) -> List[Request]:
        """Drop every request (weights changed: their KV and partial outputs are stale)."""
        dropped = self.running_queue + self.waiting_queue
        self.running_queue, self.waiting_queue = [], []
        return dropped

    def has_pending_requests(self) -> bool:
        return bool(self.waiting_queue or self.running_queue)

    def get_stats(self) -> dict:
        return {"waiting": len(self.waiting_queue), "running": len(self.running_queue),
                "total_scheduled": self.total_scheduled, "total_preempted": self.total_preempted,
                "total_finished": self.total_finished}
