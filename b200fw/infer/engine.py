"""InferenceEngine: continuous batching over the native paged model.

Public surface of the reference engine (src/inference/engine.py:197-1693): ``initialize``,
``add_request`` / ``step``, ``generate``, ``on_weights_updated``, ``has_pending``, ``get_stats``, with
three modes — ``kv_cache`` (the product path: scheduler-driven chunked prefill + batched paged decode,
prefix / radix block sharing, optional CUDA-graph decode, split-KV attention and speculative decoding),
``eager`` (full re-forward per token, the oracle) and ``mock`` (scheduler + random tokens, no model).
Per-request failures are isolated (the request is finished with what it has and its blocks are
returned); a CUDA out-of-memory error clears caches and graphs and reports ``None`` for the batch.
"""
from __future__ import annotations

import contextlib
import functools
import operator
import random
import threading
import time
from typing import Dict, List, Optional

import torch

from ..model import ModelConfig, ParallelTransformerModel, load_from_hf_checkpoint, read_hf_config
from ..obs import nvtx
from ..obs.logging import get_logger
from .config import InferenceConfig
from .graphs import CUDAGraphRunner
from .kv_cache import BlockPool, KVCacheManager
from .prefix_cache import PrefixCache
from .radix_cache import RadixAttentionCache
from .runner import ModelRunner
from .scheduler import ContinuousBatchingScheduler, Request, SchedulerOutput
from .spec import SpeculativeDecoder

def _locked(fn):
    """Run a public entry point under the engine's lock.  A rollout runs on a worker thread while the trainer's thread
    publishes new weights (``load_weights`` / ``on_weights_updated``), and a server thread may add or cancel requests:
    each of these mutates the scheduler queues, the block tables and the launch in flight, so they take turns, one
    engine step at a time.  Re-entrant (``load_weights`` calls ``on_weights_updated``); uncontended cost ~0.1 us."""
    @functools.wraps(fn)
    def inner(self, *a, **k):
        with self._lock:
            return fn(self, *a, **k)
    return inner


logger = get_logger("infer.engine")


class InferenceEngine:
    def __init__(self, config: InferenceConfig, model: Optional[ParallelTransformerModel] = None,
                 draft_model: Optional[ParallelTransformerModel] = None):
        self.config = config
        self.model = model
        self.draft_model = draft_model
        self.scheduler: Optional[ContinuousBatchingScheduler] = None
        self.pool: Optional[BlockPool] = None
        self.kv: Optional[KVCacheManager] = None
        self.runner: Optional[ModelRunner] = None
        self.prefix_cache = None
        self._inflight_prefix: Dict[tuple, str] = {}
        self.graph_runner: Optional[CUDAGraphRunner] = None
        self.spec: Optional[SpeculativeDecoder] = None
        self.requests: Dict[str, Request] = {}
        self.finished: Dict[str, Request] = {}
        self.initialized = False
        self.weights_version = 0
        self._inflight: Optional[dict] = None       # the decode launch whose sampled ids are still on the device
        self._stage_rings: dict = {}
        self._samp_cache = None
        self.stats = {"steps": 0, "prefill_tokens": 0, "decode_tokens": 0, "cached_prefix_tokens": 0,
                      "oom_recoveries": 0, "request_errors": 0, "graph_replays": 0, "spec_rounds": 0}
        self._rng = random.Random(config.seed)
        self._lock = threading.RLock()
        self._weights_event = None                  # recorded after a weight rewrite; the next step waits for it
        self._gen: Optional[torch.Generator] = None
        self.device = torch.device("cpu")

    # =================================================================================================
    def initialize(self):
        cfg = self.config
        self.scheduler = ContinuousBatchingScheduler(cfg.max_num_batched_tokens, cfg.max_num_sequences,
                                                     cfg.max_prefill_tokens, cfg.enable_chunked_prefill,
                                                     cfg.chunk_size, cfg.adaptive_chunking)
        if cfg.inference_mode == "mock":
            self.pool = BlockPool(cfg.num_blocks, cfg.block_size, cfg.num_layers, cfg.num_kv_heads, cfg.head_dim,
                                  allocate=False)
            self.kv = KVCacheManager(self.pool, cfg.block_size)
            self.initialized = True
            return self
        if self.model is None:
            self.model = self._build_model()
        p0 = next(self.model.parameters())
        self.device = p0.device
        if self.device.type == "cuda":
            from .. import _native
            _native.set_device(self.device.index or 0)
        self._gen = torch.Generator(device=self.device).manual_seed(cfg.seed)
        self.model.eval()
        if cfg.inference_mode == "eager":
            self.initialized = True
            return self
        mc = self.model.cfg
        if self.device.type == "cuda" and cfg.block_size != 16:
            raise ValueError(f"block_size={cfg.block_size}: the paged KV kernels are built for 16-token blocks")
        self.pool = BlockPool(cfg.num_blocks, cfg.block_size, mc.num_layers, mc.num_kv_heads, mc.head_dim,
                              p0.dtype, self.device, cfg.kv_cache_dtype)
        self.kv = KVCacheManager(self.pool, cfg.block_size)
        self.runner = ModelRunner(self.model, self.pool, self.kv, cfg.attention_partition_size,
                                  cfg.enable_partitioned_attention)
        self.runner.balance_splits = cfg.decode_balance_splits
        if cfg.enable_prefix_caching or cfg.use_radix_cache:
            self.prefix_cache = RadixAttentionCache(cfg.block_size, cfg.radix_cache_max_nodes) if cfg.use_radix_cache \
                else PrefixCache(cfg.block_size, cfg.max_cached_blocks)
            self.prefix_cache.on_evict = lambda bid: self.pool.free(self.pool.get_block(bid))
            if cfg.enable_prefix_reuse:
                self.scheduler.defer = self._defer_for_shared_prefix
        if cfg.enable_cuda_graph and self.device.type == "cuda":
            self.graph_runner = CUDAGraphRunner(cfg.max_num_sequences)
            self.runner.graph_runner = self.graph_runner
        if cfg.speculative_enabled:
            self._init_speculative()
        self.initialized = True
        return self

    def _build_model(self) -> ParallelTransformerModel:
        cfg = self.config
        dev = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
        if cfg.dtype == "float16":
            logger.warning("dtype float16 runs as bfloat16: the kernels are bf16-only")
        dtype = {"bfloat16": torch.bfloat16, "float32": torch.float32, "float16": torch.bfloat16}[cfg.dtype]
        if dev.type == "cpu":
            dtype = torch.float32
        if cfg.model_path:
            mc = read_hf_config(cfg.model_path)
        else:
            mc = ModelConfig(cfg.vocab_size, cfg.hidden_size, cfg.num_layers, cfg.num_heads, cfg.num_kv_heads,
                             cfg.head_dim, cfg.intermediate_size or 3 * cfg.hidden_size)
        model = ParallelTransformerModel(mc, dtype=dtype, device=dev)
        model.init_weights(cfg.seed)
        if cfg.model_path:
            load_from_hf_checkpoint(model, cfg.model_path)
        for p in model.parameters():
            p.requires_grad_(False)
        return model

    def _init_speculative(self):
        cfg, mc = self.config, self.model.cfg
        if self.draft_model is None:
            import copy
            dc = copy.deepcopy(mc)
            dc.num_layers = cfg.speculative_draft_layers
            p0 = next(self.model.parameters())
            self.draft_model = ParallelTransformerModel(dc, dtype=p0.dtype, device=p0.device)
            self.draft_model.init_weights(cfg.seed + 1)
            if cfg.speculative_draft_model_path:
                load_from_hf_checkpoint(self.draft_model, cfg.speculative_draft_model_path)
            for p in self.draft_model.parameters():
                p.requires_grad_(False)
        self.draft_model.eval()
        dmc = self.draft_model.cfg
        p0 = next(self.draft_model.parameters())
        dpool = BlockPool(self.config.num_blocks, self.config.block_size, dmc.num_layers, dmc.num_kv_heads,
                          dmc.head_dim, p0.dtype, self.device, "fp16")
        dmgr = KVCacheManager(dpool, self.config.block_size)
        self.draft_runner = ModelRunner(self.draft_model, dpool, dmgr)
        self.spec = SpeculativeDecoder(self.runner, self.draft_runner, self.config.speculative_num_tokens)

    # =================================================================================================
    @_locked
    def add_request(self, request_id: str, prompt_tokens: List[int], max_tokens: int = 512,
                    temperature: Optional[float] = None, top_p: Optional[float] = None) -> Request:
        assert self.initialized, "call initialize() first"
        prompt_tokens, max_tokens = self._check_request(request_id, prompt_tokens, max_tokens)
        return self._enqueue(request_id, prompt_tokens, max_tokens, temperature, top_p)

    @_locked
    def _enqueue(self, request_id, prompt_tokens, max_tokens, temperature, top_p) -> Request:
        t = float(self.config.temperature if temperature is None else temperature)
        p = float(self.config.top_p if top_p is None else top_p)
        if not t >= 1e-5:
            t = 0.0                 # zero, negative, vanishing (1 / t would overflow) or NaN: greedy
        p = min(max(p, 0.0), 1.0) if p == p else 1.0
        r = Request(request_id, prompt_tokens, max_tokens, t, p, eos_token_id=self.config.eos_token_id)
        r.weights_version = self.weights_version        # the version this request started under
        self.requests[request_id] = r
        self.scheduler.add_request(r)
        return r

    def _check_request(self, request_id, prompt_tokens, max_tokens: int):
        """Refuse, at submission, a request that could not be served or would harm the others: the step loop is shared
        by every request in flight, and the embedding and rotary kernels index their tables with token ids and
        positions unchecked.  Returns the prompt as a list and ``max_tokens`` shortened to what the position table
        allows."""
        prompt = [int(t) for t in prompt_tokens]
        if not prompt:
            raise ValueError(f"request {request_id!r}: empty prompt")
        try:
            max_tokens = operator.index(max_tokens)         # int, numpy integer, 0-d integer tensor
        except TypeError:
            max_tokens = -1
        if max_tokens < 0:
            raise ValueError(f"request {request_id!r}: max_tokens must be a non-negative integer")
        if request_id in self.requests:
            raise ValueError(f"request id {request_id!r} is already in flight")
        mc = getattr(self.model, "cfg", None)
        if mc is None:                      # mock mode: no model, nothing indexed
            return prompt, max_tokens
        lo, hi = min(prompt), max(prompt)
        if lo < 0 or hi >= mc.vocab_size:
            raise ValueError(f"request {request_id!r}: token id {lo if lo < 0 else hi} is outside the vocabulary "
                             f"[0, {mc.vocab_size})")
        # speculative rounds score up to k drafted tokens past the last accepted one
        room = mc.max_position_embeddings - len(prompt) - (self.config.speculative_num_tokens + 1 if self.spec else 0)
        if room < 1:
            raise ValueError(f"request {request_id!r}: a prompt of {len(prompt)} tokens leaves no room to generate "
                             f"within max_position_embeddings={mc.max_position_embeddings}")
        if max_tokens > room:
            logger.warning("request %s: max_tokens %d shortened to %d (max_position_embeddings=%d)", request_id,
                           max_tokens, room, mc.max_position_embeddings)
            max_tokens = room
        return prompt, max_tokens

    def has_pending(self) -> bool:
        return self.scheduler.has_pending_requests()

    # ---- one engine step ----------------------------------------------------------------------------------
    @_locked
    def step(self) -> Dict[str, List[int]]:
        """Schedule, run prefill chunks and one decode token for every running sequence.  Returns the
        tokens produced in this step per request id."""
        ev, self._weights_event = self._weights_event, None
        if ev is not None:
            torch.cuda.current_stream().wait_event(ev)
        with nvtx.range("infer/schedule"):
            out = self.scheduler.schedule()
        self.stats["steps"] += 1
        for r in out.preempted_requests:
            self._release(r, cache_prefix=False)
        produced: Dict[str, List[int]] = {}
        if out.preempted_requests or out.is_empty:
            self._resolve_inflight(produced)        # a preempted request's progress is reset: settle its tokens first
        if out.is_empty:
            self._finish_done(produced)
            return produced
        try:
            decode = [r for r in out.decode_requests if r.request_id not in out.prefill_tokens]
            if out.prefill_requests:
                self._resolve_inflight(produced)    # steps with prefill chunks run synchronously
                with nvtx.range("infer/prefill"):
                    self._execute_prefill(out, produced)
            if decode:
                with nvtx.range("infer/decode"):
                    self._execute_decode(decode, produced, lookahead=not out.prefill_requests)
        except torch.cuda.OutOfMemoryError:
            self._inflight = None
            self._recover_from_oom()
            return produced
        self._finish_done(produced)
        return produced

    def _finish_done(self, produced: Dict[str, List[int]]):
        """Retire requests that are complete.  A request whose last token is still on the device (sampled by the
        launch in flight) is complete by count: its values are read now, so that nothing unresolved leaves the engine."""
        inf = self._inflight
        if inf is not None and any(r.is_finished for r in inf["reqs"]):
            self._resolve_inflight(produced)
        for rid in list(produced):
            r = self.requests.get(rid)
            if r is not None and r.is_finished:
                self._finish(r)

    # ---- sampled ids that are still on the device ------------------------------------------------------------------
    PLACEHOLDER = -1

    def _resolve_inflight(self, produced: Optional[Dict[str, List[int]]] = None):
        """Read the ids (and log-probs) of the decode launch in flight into the requests' output lists (this waits
        for that launch).  An EOS found here ends its request: whatever the following launch sampled for it is
        dropped."""
        inf, self._inflight = self._inflight, None
        if inf is None:
            return
        if inf["event"] is not None:
            if inf["event"].query():
                self.stats["inflight_ready"] = self.stats.get("inflight_ready", 0) + 1    # the GPU was ahead of the host
            else:
                t0 = time.perf_counter()
                inf["event"].synchronize()
                self.stats["inflight_wait_s"] = self.stats.get("inflight_wait_s", 0.0) + time.perf_counter() - t0
                self.stats["inflight_waited"] = self.stats.get("inflight_waited", 0) + 1
        ids, lps = inf["host_ids"][:len(inf["reqs"])].tolist(), inf["host_lps"][:len(inf["reqs"])].tolist()
        for r, slot, t, lp in zip(inf["reqs"], inf["slots"], ids, lps):
            if slot >= len(r.output_tokens) or r.output_tokens[slot] != self.PLACEHOLDER:
                continue                            # the request ended (EOS) or was reset since this launch
            r.output_tokens[slot] = t
            r.output_logprobs[slot] = lp
            if produced is not None:
                produced.setdefault(r.request_id, []).append(t)
            if r.eos_token_id is not None and t == r.eos_token_id:
                del r.output_tokens[slot + 1:]
                del r.output_logprobs[slot + 1:]

    # ---- prefill --------------------------------------------------------------------------------------------
    def _first_block_key(self, r: Request):
        bs = self.config.block_size
        return tuple(r.prompt_tokens[:bs]) if r.num_prompt_tokens > bs else None

    def _defer_for_shared_prefix(self, r: Request) -> bool:
        """True while another request that starts with the same block is still prefilling: once that
        one publishes its prompt blocks, this one shares them instead of recomputing them (requests of
        one GRPO group arrive together with identical prompts)."""
        key = self._first_block_key(r)
        if key is None:
            return False
        owner = self._inflight_prefix.get(key)
        if owner is None or owner not in self.requests:
            self._inflight_prefix[key] = r.request_id      # this request computes the prefix for the others
            return False
        return owner != r.request_id

    def _admit(self, r: Request) -> bool:
        """First chunk of a request: allocate its block table, sharing cached prefix blocks."""
        shared: List[int] = []
        if self.prefix_cache is not None and self.config.enable_prefix_reuse and r.num_computed_tokens == 0:
            # never reuse the whole prompt: the last token must be computed to get logits
            matched, ids = self.prefix_cache.match_prefix(r.prompt_tokens[:-1])
            shared = ids
            r.num_cached_tokens = matched
        need = r.num_prompt_tokens
        if not self.kv.can_allocate(need - len(shared) * self.config.block_size):
            if self.prefix_cache is not None:
                self.prefix_cache.evict_lru(self.kv.blocks_needed(need))
        table = self.kv.allocate_for_sequence(r.request_id, need, shared)
        if table is None:
            if shared:
                self.prefix_cache.release_blocks(shared)
            return False
        r.num_computed_tokens = r.num_cached_tokens
        self.stats["cached_prefix_tokens"] += r.num_cached_tokens
        return True

    def _execute_prefill(self, out: SchedulerOutput, produced: Dict[str, List[int]]):
        cfg = self.config
        batch, starts, counts = [], [], []
        for r in out.prefill_requests:
            n = out.prefill_tokens[r.request_id]
            if cfg.inference_mode == "mock":
                r.num_computed_tokens += n
                if r.is_prefill_complete:
                    produced.setdefault(r.request_id, []).append(self._mock_token(r))
                continue
            try:
                if r.request_id not in self.kv.tables and not self._admit(r):
                    if self.kv.tables:
                        # other sequences hold the blocks: this one waits for them instead of failing
                        self.scheduler.requeue(r)
                        self.stats["admission_deferrals"] = self.stats.get("admission_deferrals", 0) + 1
                        continue
                    raise RuntimeError("KV cache exhausted")     # it does not fit even into an empty pool
                n = min(n, r.num_prompt_tokens - r.num_computed_tokens)   # a cached prefix shortens the chunk
                if n <= 0:
                    n = 1
                    r.num_computed_tokens = r.num_prompt_tokens - 1
                batch.append(r)
                starts.append(r.num_computed_tokens)
                counts.append(n)
            except Exception as e:  # noqa: BLE001 - isolate the failing request
                self._fail(r, e)
        if cfg.inference_mode == "mock" or not batch:
            self.stats["prefill_tokens"] += out.num_prefill_tokens
            return
        ids = [t for r, s, n in zip(batch, starts, counts) for t in r.prompt_tokens[s:s + n]]
        ctx = self.runner.prepare_prefill([r.request_id for r in batch], starts, counts)
        tok = torch.tensor(ids, dtype=torch.long)
        tok = tok.pin_memory().to(self.device, non_blocking=True) if self.device.type == "cuda" else tok
        logits = self.runner.forward(tok, ctx)
        self.stats["prefill_tokens"] += len(ids)
        done = [i for i, (r, s, n) in enumerate(zip(batch, starts, counts)) if s + n >= r.num_prompt_tokens]
        for r, n in zip(batch, counts):
            r.num_computed_tokens += n
            self.scheduler.promote_if_prefilled(r)
        if done and self.prefix_cache is not None:
            # a finished prefill's full prompt blocks are immutable from here on: publish them right away
            # so that requests admitted in later steps can share them while this one is still decoding
            for i in done:
                r = batch[i]
                if not getattr(r, "_prefix_published", False):
                    for bid in self.prefix_cache.insert(r.prompt_tokens, self.kv.get_block_table(r.request_id)):
                        self.pool.share(bid)
                    r._prefix_published = True
                    self._drop_inflight(r)
        if done:
            rows = torch.tensor(done, device=self.device)
            new, lps = self._sample([batch[i] for i in done], logits.index_select(0, rows))
            for i, t, lp in zip(done, new, lps):
                r = batch[i]
                r.output_tokens.append(t)
                r.output_logprobs.append(lp)
                produced.setdefault(r.request_id, []).append(t)
                if self.spec is not None:
                    self._draft_prefill(r)

    def _draft_prefill(self, r: Request):
        """Bring the draft model's cache level with the target's for a sequence that just finished
        prefill (whole prompt in one go: the draft is tiny)."""
        dm = self.draft_runner
        if dm.mgr.allocate_for_sequence(r.request_id, r.num_prompt_tokens) is None:
            # no room in the draft cache: this sequence simply decodes without speculation
            self.stats["spec_fallbacks"] = self.stats.get("spec_fallbacks", 0) + 1
            return
        ctx = dm.prepare_prefill([r.request_id], [0], [r.num_prompt_tokens])
        dm.forward(torch.tensor(r.prompt_tokens, dtype=torch.long, device=self.device), ctx)

    # ---- decode ---------------------------------------------------------------------------------------------
    def _execute_decode(self, reqs: List[Request], produced: Dict[str, List[int]], lookahead: bool = False):
        cfg = self.config
        if cfg.inference_mode == "mock":
            for r in reqs:
                t = self._mock_token(r)
                produced.setdefault(r.request_id, []).append(t)
            self.stats["decode_tokens"] += len(reqs)
            return
        if self.spec is not None and self._use_speculation(reqs):
            self._resolve_inflight(produced)
            return self._execute_speculative(reqs, produced)
        # a request that ended on an EOS found since scheduling needs no further token
        reqs = [r for r in reqs if not (r.output_tokens and r.output_tokens[-1] != self.PLACEHOLDER and r.is_finished)]
        live = []
        for r in reqs:
            if r.request_id not in self.kv.tables:
                continue                    # preempted a moment ago to make room for an older request
            try:
                room = self._append_token_making_room(r, live, produced)
                if room is None:
                    continue                # r itself was the newest holder of blocks: preempted, it retries later
                if not room:
                    raise RuntimeError("KV cache exhausted during decode")
                live.append(r)
            except Exception as e:  # noqa: BLE001
                self._resolve_inflight(produced)
                self._fail(r, e)
        if not live:
            return
        # on a GPU by default; "force" runs the same bookkeeping on the CPU too (tests of the one-step-late logic)
        use_async = (lookahead and bool(cfg.async_decode) and self.spec is None
                     and (self.device.type == "cuda" or cfg.async_decode == "force"))
        inf = self._inflight
        last = None
        if inf is not None:
            rows = inf["rows"]
            if use_async and all(r.request_id in rows for r in live):
                # the ids sampled by the launch in flight feed this launch straight from the device
                idx = [rows[r.request_id] for r in live]
                if idx == list(range(len(inf["reqs"]))):
                    last = inf["ids_dev"]
                else:
                    sel = self._stage("sel", torch.tensor(idx, dtype=torch.long))
                    last = inf["ids_dev"].index_select(0, sel)
            else:
                self._resolve_inflight(produced)
                live = [r for r in live if not r.is_finished] or live[:0]
                if not live:
                    return
        if last is None:
            last = self._stage("last", torch.tensor([r.output_tokens[-1] for r in live], dtype=torch.long))
        logits = self._decode_forward(live, last)
        self.stats["decode_tokens"] += len(live)
        if not use_async:
            new, lps = self._sample(live, logits[:len(live)])
            for r, t, lp in zip(live, new, lps):
                r.output_tokens.append(t)
                r.output_logprobs.append(lp)
                produced.setdefault(r.request_id, []).append(t)
            return
        ids_dev, lps_dev = self._sample_device(live, logits[:len(live)])
        n = len(live)
        if self.device.type == "cuda":
            host_ids, host_lps = self._pinned_out(n)
            host_ids[:n].copy_(ids_dev, non_blocking=True)
            host_lps[:n].copy_(lps_dev, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record()
        else:
            host_ids, host_lps, ev = ids_dev, lps_dev, None
        slots = []
        for r in live:
            slots.append(len(r.output_tokens))
            r.output_tokens.append(self.PLACEHOLDER)
            r.output_logprobs.append(0.0)
        # settle the previous launch now: the GPU finished it before it could start the one just queued, and the host
        # work of this step ran while it was executing
        self._resolve_inflight(produced)
        self._inflight = {"reqs": live, "rows": {r.request_id: i for i, r in enumerate(live)}, "slots": slots,
                          "ids_dev": ids_dev, "host_ids": host_ids, "host_lps": host_lps, "event": ev}

    def _append_token_making_room(self, r: Request, live: List[Request], produced: Dict[str, List[int]]):
        """Reserve the KV slot of ``r``'s next token.  When the pool is dry: first the prefix cache gives up blocks, then
        the newest request that holds blocks is preempted (its blocks are freed, it goes back to the head of the
        waiting queue and is recomputed later) - the policy the scheduler applies to its sequence limit, extended to
        memory (the reference preempts on the count limits only: src/inference/scheduler.py:316-339, and fails the
        request here).  Returns True (slot reserved), None (``r`` itself was the newest and has been preempted) or
        False (``r`` alone exhausts the pool: it cannot be served)."""
        while True:
            if self.kv.append_token(r.request_id):
                return True
            if self.prefix_cache is not None and self.prefix_cache.evict_lru(4):
                continue
            holders = [q for q in list(self.scheduler.running_queue) + list(self.scheduler.waiting_queue)
                       if q.request_id in self.kv.tables]
            if not holders or holders == [r]:
                return False
            victim = max(holders, key=lambda q: q.arrival_time)
            self._resolve_inflight(produced)        # placeholders of the launch in flight are settled before a reset
            self.scheduler.preempt(victim)
            self._release(victim, cache_prefix=False)
            self.stats["memory_preemptions"] = self.stats.get("memory_preemptions", 0) + 1
            if victim in live:
                live.remove(victim)
            if victim is r:
                return None

    def _stage(self, name: str, t: torch.Tensor) -> torch.Tensor:
        """Host tensor -> device through a small ring of pinned staging buffers (no page-locking per call; a ring
        because the copy of the previous step may not have run yet when this step's values are written)."""
        if self.device.type != "cuda":
            return t
        ring = self._stage_rings.setdefault((name, t.dtype), {"bufs": [None] * 4, "i": 0})
        i = ring["i"] = (ring["i"] + 1) % 4
        buf = ring["bufs"][i]
        if buf is None or buf.numel() < t.numel():
            buf = ring["bufs"][i] = torch.empty(max(256, t.numel()), dtype=t.dtype, pin_memory=True)
        view = buf[:t.numel()].view(t.shape)
        view.copy_(t)
        return view.to(self.device, non_blocking=True)

    def _pinned_out(self, n: int):
        ring = self._stage_rings.setdefault("out", {"bufs": [None] * 4, "i": 0})
        i = ring["i"] = (ring["i"] + 1) % 4
        if ring["bufs"][i] is None or ring["bufs"][i][0].numel() < n:
            ring["bufs"][i] = (torch.empty(max(256, n), dtype=torch.long, pin_memory=True),
                               torch.empty(max(256, n), dtype=torch.float32, pin_memory=True))
        return ring["bufs"][i]

    def _decode_forward(self, live: List[Request], last: torch.Tensor) -> torch.Tensor:
        ids = [r.request_id for r in live]
        gr = self.graph_runner
        if gr is None:
            return self.runner.forward(last, self.runner.prepare_decode(ids))
        size = gr.padded_size(len(live))
        width = self._graph_table_width()
        ctx = self.runner.prepare_decode(ids, pad_to=size, max_blocks=width)
        if ctx.block_tables.shape[1] > width or size is None:
            return self.runner.forward(last, self.runner.prepare_decode(ids))   # longer than the graphs cover
        plan = self._graph_split_plan(width)
        if not gr.has(size):
            def make(n):
                return {"tokens": torch.zeros(n, dtype=torch.long, device=self.device),
                        "positions": torch.zeros(n, dtype=torch.int32, device=self.device),
                        "block_tables": torch.full((n, width), -1, dtype=torch.int32, device=self.device),
                        "context_lens": torch.zeros(n, dtype=torch.int32, device=self.device),
                        "segments": torch.tensor([[-1, 0, 0, 0]] * n, dtype=torch.int32, device=self.device),
                        "slots": torch.full((n,), -1, dtype=torch.int32, device=self.device)}

            def fn(inp):
                from .context import InferenceContext
                c = InferenceContext(False, inp["tokens"].shape[0], inp["block_tables"], inp["context_lens"],
                                     width * self.config.block_size, inp["segments"], positions=inp["positions"],
                                     slot_mapping=inp["slots"])
                return self.runner.forward(inp["tokens"], c, split_plan=plan)
            gr.capture(size, make, fn)
        tokens = torch.zeros(size, dtype=torch.long, device=self.device)
        tokens[:len(live)] = last
        self.stats["graph_replays"] += 1
        return gr.replay(size, {"tokens": tokens, "positions": ctx.positions, "block_tables": ctx.block_tables,
                                "context_lens": ctx.context_lens, "segments": ctx.store_segments,
                                "slots": ctx.slot_mapping})

    def _graph_table_width(self) -> int:
        """Block-table width the graphs are captured for (grows in powers of two with the longest
        sequence; growth invalidates the captured graphs)."""
        longest = max((self.kv.get_seq_token_count(s) for s in self.kv.tables), default=1)
        need = self.kv.blocks_needed(longest + 1)
        w = getattr(self, "_graph_width", 0)
        if need > w:
            w = 64
            while w < need:
                w *= 2
            if getattr(self, "_graph_width", 0) and self.graph_runner is not None:
                self.graph_runner.invalidate()
            self._graph_width = w
        return self._graph_width

    def _graph_split_plan(self, width: int):
        if not self.config.enable_partitioned_attention:
            return (0, 1)
        part = max(64, self.config.attention_partition_size // 64 * 64)
        cap = width * self.config.block_size
        return (part, (cap + part - 1) // part) if cap > part else (0, 1)

    # ---- speculative ------------------------------------------------------------------------------------------
    def _use_speculation(self, reqs: List[Request]) -> bool:
        temps = {r.temperature for r in reqs}
        return len(temps) == 1 and all(r.request_id in self.draft_runner.mgr.tables for r in reqs) and \
            (self.spec.steps < 4 or self.spec.acceptance_rate > 0.2)

    def _execute_speculative(self, reqs: List[Request], produced: Dict[str, List[int]]):
        ids = [r.request_id for r in reqs]
        if not self.spec.can_step(ids):
            # memory is tight: give up the draft state of these sequences (they continue without speculation) and let
            # the ordinary decode step deal with the pressure (prefix-cache eviction, preemption of the newest)
            for rid in ids:
                self.draft_runner.mgr.free_sequence(rid)
            self.stats["spec_fallbacks"] = self.stats.get("spec_fallbacks", 0) + len(ids)
            return self._execute_decode(reqs, produced)
        outs = self.spec.step(ids, [r.output_tokens[-1] for r in reqs], reqs[0].temperature, self._gen)
        self.stats["spec_rounds"] += 1
        for r, toks in zip(reqs, outs):
            for t in toks:
                if r.is_finished:
                    break
                r.output_tokens.append(t)
                r.output_logprobs.append(0.0)
                produced.setdefault(r.request_id, []).append(t)
            self.stats["decode_tokens"] += len(toks)

    # ---- sampling / mock ----------------------------------------------------------------------------------------
    def _sampling_params(self, reqs: List[Request]):
        """Per-row temperature / top-p on the device, rebuilt only when the batch changes."""
        key = tuple((r.request_id, r.temperature, r.top_p) for r in reqs)
        if self._samp_cache is None or self._samp_cache[0] != key:
            both = self._stage("samp", torch.tensor([[r.temperature for r in reqs], [r.top_p for r in reqs]],
                                                    dtype=torch.float32))
            self._samp_cache = (key, both[0].contiguous(), both[1].contiguous())
        return self._samp_cache[1], self._samp_cache[2]

    def _sample_device(self, reqs: List[Request], logits: torch.Tensor):
        temp, topp = self._sampling_params(reqs)
        return self.runner.sample(logits.contiguous(), temp, topp, self._gen, return_logprob=True)

    def _sample(self, reqs: List[Request], logits: torch.Tensor):
        ids, lps = self._sample_device(reqs, logits)
        return ids.tolist(), lps.tolist()

    def _mock_token(self, r: Request) -> int:
        lo = 3 if self.config.vocab_size > 4 else 0
        t = self._rng.randrange(lo, self.config.vocab_size)
        r.output_tokens.append(t)
        return t

    # ---- lifecycle ------------------------------------------------------------------------------------------------
    def _drop_inflight(self, r: Request):
        key = self._first_block_key(r)
        if key is not None and self._inflight_prefix.get(key) == r.request_id:
            del self._inflight_prefix[key]

    def _release(self, r: Request, cache_prefix: bool = True):
        self._drop_inflight(r)
        if self.kv is None or r.request_id not in self.kv.tables:
            return
        table = self.kv.get_block_table(r.request_id)
        if cache_prefix and self.prefix_cache is not None and r.is_prefill_complete \
                and not getattr(r, "_prefix_published", False):
            for bid in self.prefix_cache.insert(r.prompt_tokens, table):
                self.pool.share(bid)            # the cache holds its own reference
        if self.prefix_cache is not None and r.num_cached_tokens:
            self.prefix_cache.release_blocks(table[:r.num_cached_tokens // self.config.block_size])
        self.kv.free_sequence(r.request_id)
        if self.spec is not None:
            self.draft_runner.mgr.free_sequence(r.request_id)

    def _finish(self, r: Request):
        self._release(r)
        self.scheduler.finish_request(r.request_id)
        self.finished[r.request_id] = r
        self.requests.pop(r.request_id, None)

    @_locked
    def abort_request(self, request_id: str) -> bool:
        """Take one request out of the engine (its client went away): the tokens it has are settled (a launch in
        flight is read first, so no placeholder is left behind), its blocks go back to the pool (a finished prompt is
        still published to the prefix cache), and it is handed over in ``finished`` with what it produced.  Returns
        False when no such request is in flight.  The reference has no cancellation: a request runs to its token
        limit (src/inference/engine.py:478-497)."""
        r = self.requests.get(request_id)
        if r is None:
            return False
        self._resolve_inflight()
        if self.PLACEHOLDER in r.output_tokens:      # defensive: nothing unread may leave the engine
            cut = r.output_tokens.index(self.PLACEHOLDER)
            del r.output_tokens[cut:]
            del r.output_logprobs[cut:]
        r.max_tokens = r.num_generated_tokens
        self.stats["aborted_requests"] = self.stats.get("aborted_requests", 0) + 1
        self._finish(r)
        return True

    def _fail(self, r: Request, err: Exception):
        logger.warning("request %s failed: %s", r.request_id, err)
        self.stats["request_errors"] += 1
        r.max_tokens = r.num_generated_tokens      # finished with what it has
        self._finish(r)

    def _recover_from_oom(self):
        logger.warning("CUDA out of memory: clearing KV cache, prefix cache and graphs")
        self.stats["oom_recoveries"] += 1
        for r in self.scheduler.abort_all():
            # ids the abandoned launch would have produced were never read: the request ends before them
            if self.PLACEHOLDER in r.output_tokens:
                cut = r.output_tokens.index(self.PLACEHOLDER)
                del r.output_tokens[cut:]
                del r.output_logprobs[cut:]
            self.finished[r.request_id] = r
            self.requests.pop(r.request_id, None)
        if self.prefix_cache is not None:
            self.prefix_cache.invalidate_all()
        self._inflight_prefix.clear()
        if self.kv is not None:
            self.kv.reset()
        if self.spec is not None:
            self.draft_runner.mgr.reset()
        if self.graph_runner is not None:
            self.graph_runner.invalidate()
        if torch.cuda.is_available():
            torch.cuda.empty_cache()

    # =================================================================================================
    def generate(self, prompts_tokens: List[List[int]], max_tokens: int = 128, temperature: Optional[float] = None,
                 top_p: Optional[float] = None, return_logprobs: bool = False):
        """Generate for a batch of prompts; returns the output token lists in prompt order (``None`` for
        a prompt whose request was dropped by an out-of-memory recovery)."""
        assert self.initialized
        base = f"gen{time.monotonic_ns()}"
        # all or nothing: nothing is queued (or computed) if one prompt is bad
        checked = [self._check_request(f"{base}-{i}", p, max_tokens) for i, p in enumerate(prompts_tokens)]
        if self.config.inference_mode == "eager":
            return self._generate_eager(checked, temperature, top_p)
        rids = []
        for i, (p, mt) in enumerate(checked):
            rid = f"{base}-{i}"
            self._enqueue(rid, p, mt, temperature, top_p)
            rids.append(rid)
        guard = 0
        limit = (max_tokens + 8) * (len(prompts_tokens) + 8) + sum(len(p) for p in prompts_tokens)
        while any(r in self.requests for r in rids):
            self.step()
            guard += 1
            if guard > limit:
                raise RuntimeError("generate() made no progress")
        outs, lps = [], []
        for rid in rids:
            r = self.finished.pop(rid, None)
            outs.append(None if r is None else list(r.output_tokens))
            lps.append(None if r is None else list(r.output_logprobs))
        return (outs, lps) if return_logprobs else outs

    @torch.no_grad()
    def _generate_eager(self, checked, temperature, top_p):
        """Full re-forward per token, no KV cache: slow, simple, and the oracle for the paged path.  ``checked``:
        ``(prompt, max_tokens)`` pairs from :meth:`_check_request`."""
        from ..ops import topp_sample
        t = self.config.temperature if temperature is None else temperature
        p = self.config.top_p if top_p is None else top_p
        outs = []
        for prompt, max_tokens in checked:
            seq, new = list(prompt), []
            for _ in range(max_tokens):
                ids = torch.tensor([seq], dtype=torch.long, device=self.device)
                logits = self.model(ids)[:, -1, :].float().contiguous()
                u = torch.rand(1, device=self.device, generator=self._gen)
                tok = int(topp_sample(logits, torch.tensor([t], device=self.device),
                                      torch.tensor([p], device=self.device), u))
                new.append(tok)
                seq.append(tok)
                if self.config.eos_token_id is not None and tok == self.config.eos_token_id:
                    break
            outs.append(new)
        return outs

    # ---- weight updates --------------------------------------------------------------------------------------------
    @contextlib.contextmanager
    def paused(self):
        """``with engine.paused():`` - no engine step runs inside the block, and the launch in flight (the one-step-late
        decode) has been read, so nothing of this engine is executing on the device: the place to rewrite the live
        weights in place from another thread.  Follow it with :meth:`on_weights_updated`."""
        with self._lock:
            self._resolve_inflight()
            yield self

    @_locked
    @torch.no_grad()
    def load_weights(self, named_tensors) -> int:
        """Copy HF-named tensors into the live model *in place* (captured graphs keep working)."""
        from ..model.hf_io import hf_named_tensors
        mine = dict(hf_named_tensors(self.model))
        n = 0
        self._resolve_inflight()            # the launch in flight reads the weights: let it finish first
        for k, v in (named_tensors.items() if isinstance(named_tensors, dict) else named_tensors):
            if k in mine:
                mine[k].copy_(v.to(mine[k].dtype))
                n += 1
        self.on_weights_updated()
        return n

    @_locked
    def on_weights_updated(self, abort_running: Optional[bool] = None):
        """The live weights changed (in place, so captured graphs stay valid).  Running requests keep decoding:
        the K/V of their earlier tokens came from the previous version, which is bounded staleness, not an error.
        A request is dropped only when it started more than ``config.max_weight_staleness`` versions ago (or when
        ``abort_running`` says so).  The prefix cache is emptied either way: no new request may share blocks
        computed under old weights."""
        self._resolve_inflight()
        self.weights_version += 1
        if self.device.type == "cuda":
            # the rewrite was queued on the caller's stream; the next step may run on another one (the rollout stream
            # of a worker thread) and must not start before the new weights have landed
            self._weights_event = torch.cuda.Event()
            self._weights_event.record()
        limit = self.config.max_weight_staleness
        abort_all = abort_running if abort_running is not None else limit <= 0
        if self.scheduler is not None:
            if abort_all:
                dropped = self.scheduler.abort_all()
            else:
                too_old = lambda r: self.weights_version - getattr(r, "weights_version", self.weights_version) > limit
                dropped = [r for r in self.scheduler.running_queue + self.scheduler.waiting_queue if too_old(r)]
                self.scheduler.running_queue = [r for r in self.scheduler.running_queue if not too_old(r)]
                self.scheduler.waiting_queue = [r for r in self.scheduler.waiting_queue if not too_old(r)]
            for r in dropped:
                self._release(r, cache_prefix=False)
                self.finished[r.request_id] = r
                self.requests.pop(r.request_id, None)
            self.stats["aborted_stale"] = self.stats.get("aborted_stale", 0) + len(dropped)
        if self.prefix_cache is not None:
            self.prefix_cache.invalidate_all()
            self._inflight_prefix.clear()
            # blocks of still-running requests stay theirs; they are never published to the cache again
            for r in (self.scheduler.running_queue if self.scheduler is not None else []):
                r._prefix_published = True
                r.num_cached_tokens = 0

    def get_stats(self) -> dict:
        s = dict(self.stats)
        s["weights_version"] = self.weights_version
        if self.scheduler is not None:
            s["scheduler"] = self.scheduler.get_stats()
        if self.kv is not None:
            s["kv_cache"] = self.kv.get_stats()
        if self.prefix_cache is not None:
            s["prefix_cache"] = self.prefix_cache.get_stats()
        if self.graph_runner is not None:
            s["cuda_graphs"] = self.graph_runner.get_stats()
        if self.spec is not None:
            s["speculative"] = {"acceptance_rate": self.spec.acceptance_rate, "rounds": self.spec.steps}
        return s
