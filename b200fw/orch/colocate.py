"""Colocate orchestrator: SFT or GRPO iterations with rollout, reward, training and weight sync on the
same set of GPUs.

State machine and artefacts follow the reference (src/orchestrator/colocate_orchestrator.py:43-1848):
``INIT -> [INFERRING -> REWARDING -> TRAINING -> SLEEPING -> SYNCING]* -> DONE`` (``ERROR`` on a failed
iteration, after which the loop carries on), per-iteration JSONL rows, ``run_summary.json``,
``config_snapshot.json``, ``loss_curve.csv``, memory timeline / report, optional TensorBoard scalars,
``iter_N`` / ``latest`` / ``final`` checkpoints, MFU sampling.  Rollouts run in the native paged
engine of this process (the reference's "custom" backend generates with the trainer model, one
sequence at a time and without a KV cache); the vLLM server backend is kept behind the same interface.
With ``async_pipeline`` the rollout for iteration N+1 overlaps the training of iteration N on a worker
thread and a second CUDA stream, and rollouts older than ``max_staleness`` weight versions are dropped
and regenerated — the reference declares that knob but never enforces it.
"""
from __future__ import annotations

import asyncio
import csv
import enum
import json
import math
import os
import time
from concurrent.futures import ThreadPoolExecutor
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch

from ..config import ColocateConfig, config_snapshot
from ..dist.heartbeat import PeerLostError
from ..data import GRPOBatch, GSM8KDataPipeline, SyntheticTokenPipeline
from ..infer import InferenceConfig, InferenceEngine
from ..obs import (ArtifactWriter, CommProfiler, ComputeProfiler, EvalMetrics, MemoryProfiler, MetricsCollector,
                   compute_bleu4, compute_exact_match, compute_token_f1, get_logger)
from ..reward import GSM8KRewardFunction, SyntheticTokenReward
from ..sync import PeerWeightSync, SwiftSyncConfig, SwiftSyncTransfer
from ..train import C3POConfig, C3POPlusScheduler, TrainConfig, TrainEngine, TrainMetrics

logger = get_logger("orch.colocate")


class OrchestratorState(enum.Enum):
    INIT = "init"
    TRAINING = "training"
    SLEEPING = "sleeping"
    SYNCING = "syncing"
    INFERRING = "inferring"
    REWARDING = "rewarding"
    ERROR = "error"
    DONE = "done"


@dataclass
class IterationMetrics:
    iteration: int
    state_durations: Dict[str, float] = field(default_factory=dict)
    train_metrics: Optional[TrainMetrics] = None
    avg_reward: float = 0.0
    accuracy: float = 0.0
    iteration_accuracy: float = 0.0
    cumulative_accuracy: float = 0.0
    total_time: float = 0.0
    tokens_generated: int = 0
    tokens_trained: int = 0
    weights_version: int = 0
    rollout_staleness: int = 0
    error: Optional[str] = None


@dataclass
class _Rollout:
    batch: GRPOBatch
    responses: List[List[List[int]]]             # [B][K][tokens]
    logprobs: Optional[List[List[float]]]        # mean per-token log-prob per response, flattened B*K
    weights_version: int
    seconds: float
    token_logprobs: Optional[List[List[List[float]]]] = None     # per-token log-probs, [prompt][sample][token]


class ColocateOrchestrator:
    def __init__(self, config: ColocateConfig, engine: Optional[TrainEngine] = None,
                 inference_engine: Optional[InferenceEngine] = None, data=None, reward_fn=None, vllm_client=None):
        self.config = config
        self.state = OrchestratorState.INIT
        self.train_engine = engine
        self.infer_engine = inference_engine
        self.data = data
        self.reward_fn = reward_fn
        self.vllm_client = vllm_client
        self.metrics: List[IterationMetrics] = []
        self.collector = MetricsCollector()
        self.memory = MemoryProfiler()
        self.comm_profiler: Optional[CommProfiler] = None
        self.compute_profiler: Optional[ComputeProfiler] = None
        self.artifacts: Optional[ArtifactWriter] = None
        self.c3po: Optional[C3POPlusScheduler] = None
        self.swift: Optional[SwiftSyncTransfer] = None
        self.weight_sync: Optional[PeerWeightSync] = None
        self.tb = None
        self._eval_snapshots: Dict[str, List[Dict]] = {}
        self.eval_results: Dict[str, Dict] = {}
        self.last_preview: Optional[str] = None
        self._last_checkpoint_path: Optional[str] = None
        self.state_log: List[str] = []
        self.weights_version = 0
        self._batches = None
        self.start_iteration = 0        # > 0 after a resume from a checkpoint that recorded its iteration
        self._resume_rng_from: Optional[str] = None
        self._stop_requested = False
        self.stopped_early = False      # the loop ended on request_stop() before total_iterations
        self._skip_batches = 0          # batches the resumed run's completed iterations had consumed
        self._pool = ThreadPoolExecutor(max_workers=1)
        self._rollout_stream = None
        self._tp_exchange_group = None
        self.ipc = None
        self._start_time = 0.0

    # ---- state --------------------------------------------------------------------------------------------
    def _set_state(self, s: OrchestratorState):
        self.state = s
        self.state_log.append(s.value)

    # =================================================================================================
    async def initialize(self):
        cfg = self.config
        if self.train_engine is None:
            total_steps = max(1, cfg.total_iterations * cfg.train_steps_per_iteration // max(1, cfg.gradient_accumulation_steps))
            tc = TrainConfig(
                model_path=cfg.model_path if cfg.model_preset is None else "", model_preset=cfg.model_preset,
                tp_size=cfg.tp_size, dp_size=cfg.dp_size, pp_size=cfg.pp_size, num_micro_batches=cfg.num_micro_batches,
                max_seq_len=cfg.max_seq_len, use_flash_attn=cfg.use_flash_attn, attention_backend=cfg.attention_backend,
                use_gradient_checkpoint=cfg.use_gradient_checkpoint, lora_rank=cfg.lora_rank, lora_alpha=cfg.lora_alpha,
                lora_target_modules=list(cfg.lora_target_modules), learning_rate=cfg.learning_rate,
                weight_decay=cfg.weight_decay, max_grad_norm=cfg.max_grad_norm, use_amp=cfg.amp_dtype != "fp32",
                amp_dtype=cfg.amp_dtype, gradient_accumulation_steps=cfg.gradient_accumulation_steps,
                grpo_num_samples=cfg.num_samples_per_prompt, grpo_beta=cfg.grpo_beta if cfg.training_mode == "grpo" else 0.0,
                grpo_clip_eps=cfg.grpo_clip_eps, zero_stage=cfg.zero_stage, enable_comm_overlap=cfg.enable_comm_overlap,
                lr_scheduler_type=cfg.lr_scheduler_type, warmup_steps=cfg.warmup_steps, min_lr_ratio=cfg.min_lr_ratio,
                total_training_steps=total_steps, icepop_enabled=cfg.icepop_enabled,
                icepop_divergence_threshold=cfg.icepop_divergence_threshold,
                icepop_max_mask_ratio=cfg.icepop_max_mask_ratio, sequence_parallel=cfg.sequence_parallel, seed=cfg.seed,
                heartbeat_interval_s=cfg.heartbeat_interval_s, heartbeat_timeout_s=cfg.heartbeat_timeout_s)
            self.train_engine = TrainEngine(tc).initialize()
        eng = self.train_engine
        eng.metrics_collector = self.collector
        ctx = eng.parallel_ctx
        self.artifacts = ArtifactWriter(cfg.output_dir, ctx.global_rank, ctx.world_size)
        self.artifacts.write_json("config_snapshot.json", config_snapshot(cfg))
        if cfg.resume_from:
            ok = eng.load_checkpoint(cfg.resume_from)
            logger.info("resume from %s: %s", cfg.resume_from, "ok" if ok else "failed")
            if ok:
                self._resume_position(cfg.resume_from)
        # ---- data + reward ----------------------------------------------------------------------------------
        if self.data is None:
            if cfg.synthetic_data:
                self.data = SyntheticTokenPipeline(eng.model_config.vocab_size, cfg.max_data_samples,
                                                   cfg.synthetic_prompt_len, cfg.seed, ctx.dp_rank, ctx.dp_size,
                                                   response_len=cfg.max_tokens if cfg.training_mode == "sft" else 0)
            else:
                self.data = GSM8KDataPipeline(
                    tokenizer_name=cfg.model_path, dataset_name=cfg.dataset_name, dataset_config=cfg.dataset_config,
                    split=cfg.dataset_split, max_samples=cfg.max_data_samples, prompt_template=cfg.prompt_template,
                    prompt_field=cfg.prompt_field, input_field=cfg.input_field or "input",
                    response_field=cfg.response_field, answer_field=cfg.answer_field or "answer",
                    dp_rank=ctx.dp_rank, dp_size=ctx.dp_size)
        if isinstance(self.data, GSM8KDataPipeline):
            tok = self.data.tokenizer
            try:
                tok_vocab = len(tok)
            except TypeError:
                tok_vocab = int(getattr(tok, "vocab_size", 0) or 0)
            if tok_vocab > eng.model_config.vocab_size:
                # fail here, once, with the reason - not in every iteration when a prompt's id is refused
                raise ValueError(f"the tokenizer has {tok_vocab} ids but the model's vocabulary is "
                                 f"{eng.model_config.vocab_size}: its prompts cannot be embedded (wrong model / "
                                 "tokenizer pair, or a preset too small for text data)")
        if self.reward_fn is None:
            self.reward_fn = SyntheticTokenReward(eng.model_config.vocab_size, cfg.seed,
                                                  dense_weight=cfg.synthetic_reward_dense_weight) if cfg.synthetic_data \
                else GSM8KRewardFunction(correct=cfg.reward_correct, wrong=cfg.reward_format, no_answer=cfg.reward_wrong)
        # ---- rollout backend ----------------------------------------------------------------------------------
        if cfg.training_mode == "grpo" or cfg.inference_preview_enabled:
            await self._init_inference()
        if cfg.c3po_plus_enabled:
            self.c3po = C3POPlusScheduler(C3POConfig(True, cfg.c3po_plus_token_budget,
                                                     cfg.c3po_plus_target_batch_tokens, cfg.c3po_plus_packing_strategy))
        if cfg.swift_sync_enabled and cfg.lora_rank > 0:
            self.swift = SwiftSyncTransfer(_LoRAWorker(self), SwiftSyncConfig(True, cfg.swift_sync_fallback_full_every,
                                                                              cfg.swift_sync_double_buffer))
        if cfg.enable_profiling:
            self.comm_profiler = CommProfiler()
            self.compute_profiler = ComputeProfiler()
        if cfg.tensorboard and ctx.is_main:
            from ..obs.tb_events import open_writer
            self.tb = open_writer(os.path.join(cfg.output_dir, "tensorboard"))
        self.memory.snapshot("init")
        return self

    async def _init_inference(self):
        cfg, eng = self.config, self.train_engine
        backend = cfg.inference_backend
        if self.infer_engine is not None:
            return
        if backend == "vllm":
            from ..sync import IPCWeightTransfer, VLLMClient
            if self.vllm_client is None:
                self.vllm_client = VLLMClient(cfg.vllm_url, max_retries=cfg.max_retries, backoff_s=cfg.retry_delay)
            if self.ipc is None:
                self.ipc = IPCWeightTransfer(self.vllm_client, cfg.ipc_chunk_size)
            self._ensure_tp_exchange_group()
            return
        mc = eng.model_config
        # pipeline parallelism: every stage holds a slice of the layers, rollouts are not served (the reference allows
        # PP for SFT only).  Tensor parallelism: every rank keeps a full single-GPU copy for its rollout engine (the
        # weights fit) and the ranks of a TP group split the group's prompts between them.
        if backend == "mock" or eng.parallel_ctx.pp_size > 1:
            ic = InferenceConfig.from_model_config(mc, inference_mode="mock", temperature=cfg.temperature, top_p=cfg.top_p)
            self.infer_engine = InferenceEngine(ic).initialize()
            return
        kw = dict(inference_mode="kv_cache", temperature=cfg.temperature, top_p=cfg.top_p,
                  kv_cache_dtype=cfg.kv_cache_dtype, enable_cuda_graph=cfg.enable_cuda_graph,
                  use_radix_cache=cfg.use_radix_cache, enable_prefix_caching=cfg.use_radix_cache,
                  max_num_batched_tokens=8192, max_prefill_tokens=4096, chunk_size=512, seed=cfg.seed,
                  # every sample of the iteration's prompts decodes concurrently when the pool has room for it (one
                  # decode wave instead of two halves the number of engine steps of a rollout)
                  max_num_sequences=max(256, min(1024, self._per_rank_batch() * cfg.num_samples_per_prompt)))
        if cfg.kv_num_blocks > 0:
            ic = InferenceConfig.from_model_config(mc, num_blocks=cfg.kv_num_blocks, **kw)
        else:
            auto = InferenceConfig.auto_from_device(mc.num_layers, mc.num_kv_heads, mc.head_dim, gpu_memory_fraction=0.3,
                                                    kv_cache_dtype=cfg.kv_cache_dtype)
            ic = InferenceConfig.from_model_config(mc, num_blocks=auto.num_blocks, **kw)
        pctx = eng.parallel_ctx
        self._ensure_tp_exchange_group()
        # one path for every layout: export (adapters merged, TP shards gathered, ZeRO-3 shards collected) into a
        # fresh single-GPU model
        rollout_model = self._merged_clone()
        self.infer_engine = InferenceEngine(ic, rollout_model).initialize()
        from ..model.hf_io import hf_named_tensors
        layout = [(k, tuple(v.shape)) for k, v in hf_named_tensors(rollout_model)]
        self.weight_sync = PeerWeightSync(layout, next(rollout_model.parameters()).dtype, eng.device)
        if torch.cuda.is_available():
            self._rollout_stream = torch.cuda.Stream()
        self._restore_rollout_rng()

    def _rollout_rng_file(self, path: str) -> str:
        return os.path.join(path, f"rollout_rng_rank{self.train_engine.parallel_ctx.global_rank}.pt")

    def _save_rollout_rng(self, path: str):
        """The sampling state of this rank's rollout engine (its device generator and the host generator of the mock
        mode) beside the checkpoint: a resumed run then draws the samples the uninterrupted run would have drawn."""
        e = self.infer_engine
        if e is None or getattr(e, "_gen", None) is None:
            return
        self.train_engine._atomic_save({"generator": e._gen.get_state().cpu(), "python": e._rng.getstate(),
                                        "weights_version": e.weights_version}, self._rollout_rng_file(path))

    def _restore_rollout_rng(self):
        path, self._resume_rng_from = self._resume_rng_from, None
        e = self.infer_engine
        if path is None or e is None or getattr(e, "_gen", None) is None:
            return
        f = self._rollout_rng_file(path)
        if not os.path.exists(f):
            return
        try:
            st = torch.load(f, map_location="cpu", weights_only=False)
            e._gen.set_state(st["generator"])
            e._rng.setstate(st["python"])
            e.weights_version = int(st.get("weights_version", e.weights_version))
        except Exception as err:  # noqa: BLE001 - a state from another device type or torch version: sample afresh
            logger.warning("resume: rollout sampling state in %s not restored (%s)", f, err)

    def _ensure_tp_exchange_group(self):
        """A group of its own (gloo: plain host objects) for handing rollouts round the TP group, so that the
        exchange - which may run on the rollout worker thread - never interleaves with training collectives."""
        pctx = self.train_engine.parallel_ctx
        if pctx.tp_size <= 1 or self._tp_exchange_group is not None:
            return
        import torch.distributed as dist
        tp_groups, _, _ = pctx.group_table(pctx.world_size, pctx.tp_size, pctx.dp_size, pctx.pp_size)
        for ranks in tp_groups:
            g = dist.new_group(ranks, backend="gloo")
            if pctx.global_rank in ranks:
                self._tp_exchange_group = g

    def _merged_clone(self):
        """Plain single-GPU copy of the policy: adapters merged in, tensor-parallel shards gathered (every rank of
        the TP group takes part in the gather), ZeRO-3 shards collected."""
        from ..model import ParallelTransformerModel
        from ..model.hf_io import hf_named_tensors
        eng = self.train_engine
        m = ParallelTransformerModel(eng.model_config, dtype=eng.dtype, device=eng.device)
        src = eng.export_weights()
        with torch.no_grad():
            for k, v in hf_named_tensors(m):
                v.copy_(src[k])
        for p in m.parameters():
            p.requires_grad_(False)
        return m

    # =================================================================================================
    def _resume_position(self, path: str):
        """Continue the run where the checkpoint left it: ``orchestrator_state.json`` (written by
        :meth:`_save_checkpoint`) names the iterations that were complete; the loop starts after them and the data
        stream skips the batches they consumed, so a resumed run sees the batches the uninterrupted one would have.  A
        checkpoint without that file (one made by ``TrainEngine.save_checkpoint`` alone, or by the reference), or one
        that already covers ``total_iterations``, restores the engine only and the loop runs from iteration 0, as the
        reference's does
        (src/orchestrator/colocate_orchestrator.py:267-272)."""
        f = os.path.join(path, "orchestrator_state.json")
        if not os.path.exists(f):
            return
        try:
            with open(f) as fh:
                st = json.load(fh)
            done = int(st.get("iterations_completed", 0))
        except (OSError, ValueError, TypeError) as e:
            logger.warning("resume: %s is unreadable (%s): starting at iteration 0", f, e)
            return
        if done >= self.config.total_iterations:
            # the checkpoint of a finished (or longer) run: a warm start, ``total_iterations`` more from its weights
            logger.info("resume: the checkpoint covers %d iterations (total_iterations is %d): warm start, the loop "
                        "runs from iteration 0", done, self.config.total_iterations)
            return
        self.start_iteration = max(0, done)
        self._skip_batches = max(0, int(st.get("batches_consumed", done)))
        self.weights_version = int(st.get("weights_version", 0))
        self._resume_rng_from = path
        logger.info("resume: continuing at iteration %d of %d", self.start_iteration, self.config.total_iterations)

    def _next_batch(self) -> GRPOBatch:
        while self._skip_batches > 0:           # resumed run: pass over what the completed iterations consumed
            self._skip_batches -= 1
            self._next_batch_raw()
        return self._next_batch_raw()

    def _next_batch_raw(self) -> GRPOBatch:
        if self._batches is None:
            self._batches = iter(self.data.get_batches(self._per_rank_batch()))
        try:
            return next(self._batches)
        except StopIteration:
            self._batches = iter(self.data.get_batches(self._per_rank_batch()))
            try:
                return next(self._batches)
            except StopIteration:
                raise ValueError(f"this rank's data shard has {len(self.data)} samples, fewer than its batch of "
                                 f"{self._per_rank_batch()}: lower training.batch_size or raise data.max_samples") from None

    def _rollout(self, batch: GRPOBatch) -> _Rollout:
        """K sampled responses per prompt through the rollout backend."""
        cfg = self.config
        t0 = time.perf_counter()
        K = cfg.num_samples_per_prompt
        prompts = [p for p in batch.prompt_tokens for _ in range(K)]
        version = self.weights_version
        ctx = self.train_engine.parallel_ctx
        share = ctx.tp_size > 1 and self.infer_engine.config.inference_mode != "mock"
        mine = list(range(ctx.tp_rank, len(prompts), ctx.tp_size)) if share else list(range(len(prompts)))
        local = [prompts[i] for i in mine]
        if self._rollout_stream is not None:
            self._rollout_stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self._rollout_stream):
                outs, lps = self.infer_engine.generate(local, cfg.max_tokens, cfg.temperature, cfg.top_p, return_logprobs=True)
            self._rollout_stream.synchronize()
        else:
            outs, lps = self.infer_engine.generate(local, cfg.max_tokens, cfg.temperature, cfg.top_p, return_logprobs=True)
        if share:
            # the ranks of a TP group train on the same batch: exchange the token ids each one generated
            import torch.distributed as dist
            parts = [None] * ctx.tp_size
            dist.all_gather_object(parts, (mine, outs, lps), group=self._tp_exchange_group)
            outs, lps = [None] * len(prompts), [None] * len(prompts)
            for idx, o, l in parts:
                for j, i in enumerate(idx):
                    outs[i], lps[i] = o[j], (l[j] if l is not None else None)
        outs = [o if o else [0] for o in outs]
        responses = [outs[i * K:(i + 1) * K] for i in range(len(batch.prompt_tokens))]
        seq_lp = [sum(l) / max(1, len(l)) if l else 0.0 for l in lps] if lps and lps[0] is not None else None
        tok_lp = None
        if seq_lp is not None and all(l is not None for l in lps):
            tok_lp = [lps[i * K:(i + 1) * K] for i in range(len(batch.prompt_tokens))]
        return _Rollout(batch, responses, seq_lp, version, time.perf_counter() - t0, tok_lp)

    async def _rollout_vllm(self, batch: GRPOBatch) -> _Rollout:
        """Rollouts from a vLLM server: K text completions per prompt over HTTP, tokenised for the trainer.  The
        server reports no per-token log-probabilities here, so IcePop recomputes the rollout policy's on the trainer."""
        cfg, t0 = self.config, time.perf_counter()
        tok = self.data.tokenizer
        version = self.weights_version
        responses = []
        pctx = self.train_engine.parallel_ctx
        if pctx.tp_rank == 0:       # one query per TP group; its other ranks receive the answers below
            for prompt in batch.prompts:
                texts = await self.vllm_client.completions(prompt, cfg.num_samples_per_prompt, cfg.max_tokens,
                                                           cfg.temperature, cfg.top_p, cfg.model_path or None)
                texts = (texts + [""] * cfg.num_samples_per_prompt)[:cfg.num_samples_per_prompt]
                responses.append([list(tok.encode(t)) or [getattr(tok, "eos_token_id", 0) or 0] for t in texts])
        if pctx.tp_size > 1:
            import torch.distributed as dist
            box = [responses]
            dist.broadcast_object_list(box, src=pctx.tp_ranks[0], group=self._tp_exchange_group)
            responses = box[0]
        return _Rollout(batch, responses, None, version, time.perf_counter() - t0)

    def _uses_vllm(self) -> bool:
        return self.vllm_client is not None and self.infer_engine is None

    def _rewards(self, ro: _Rollout) -> List[List[float]]:
        if isinstance(self.reward_fn, SyntheticTokenReward):
            return self.reward_fn(ro.responses, ro.batch.prompt_indices or list(range(len(ro.responses))))
        tok = self.data.tokenizer
        texts = [[tok.decode(r) for r in group] for group in ro.responses]
        return self.reward_fn(texts, ro.batch.ground_truths)

    def _train_grpo(self, ro: _Rollout, rewards: List[List[float]]) -> TrainMetrics:
        cfg, eng = self.config, self.train_engine
        prompts = ro.batch.prompt_tokens
        infer_lp = torch.tensor(ro.logprobs) if (ro.logprobs is not None and cfg.icepop_enabled) else None
        if self.c3po is not None:
            adv = [TrainEngine.group_advantages(r) for r in rewards]
            subs = self.c3po.split_and_pack(prompts, ro.responses, rewards, adv,
                                            ro.token_logprobs if cfg.icepop_enabled else None)
            m = None
            for i, sb in enumerate(subs):
                last = i == len(subs) - 1
                m = eng.grpo_step(**sb, skip_optimizer_step=not last, reset_behavior_baseline=True, close_window=last)
            return m
        m = None
        for s in range(cfg.train_steps_per_iteration):
            m = eng.grpo_step(prompts, ro.responses, rewards, infer_log_probs=infer_lp,
                              reset_behavior_baseline=(s == 0))
        return m

    def _train_sft(self, batch: GRPOBatch) -> TrainMetrics:
        eng = self.train_engine
        if isinstance(self.data, SyntheticTokenPipeline):
            responses = [self.data.responses[i] or [3] for i in batch.prompt_indices]
        else:
            tok = self.data.tokenizer
            responses = [tok.encode(r) + [getattr(tok, "eos_token_id", 2) or 2] for r in batch.reference_responses]
        m = None
        for _ in range(self.config.train_steps_per_iteration):
            m = eng.sft_step(batch.prompt_tokens, responses)
        return m

    def _sync_weights(self, iteration: int) -> int:
        """Publish the trainer's current weights to the rollout engine.  LoRA + SwiftSync: deltas (full
        every N); otherwise the merged full weights through the peer-write path."""
        eng = self.train_engine
        if self.infer_engine is None or self.infer_engine.config.inference_mode == "mock":
            if self.infer_engine is not None:
                self.infer_engine.on_weights_updated()
            self.weights_version += 1
            return self.weights_version
        if self.swift is not None:
            from ..model.lora import flat_lora_state
            with eng.optimizer.eval_mode():          # ZeRO-3 keeps the adapters sharded between steps: gather to read
                state = flat_lora_state(eng.model)
            self.swift.sync(iteration, state)
        else:
            state = eng.export_weights()
            self.weight_sync.sync(True, state, self.infer_engine)
        self.weights_version += 1
        return self.weights_version

    # =================================================================================================
    async def run(self) -> List[IterationMetrics]:
        cfg = self.config
        self._start_time = time.time()
        if self._stages_overridden():
            return await self._run_staged()
        loop = asyncio.get_running_loop()
        pending: Optional[asyncio.Future] = None
        if cfg.eval_num_prompts > 0 and self.start_iteration == 0:
            self._do_eval("before")
        for it in range(self.start_iteration, cfg.total_iterations):
            im = IterationMetrics(it)
            t_iter = time.perf_counter()
            try:
                if cfg.training_mode == "sft":
                    self._set_state(OrchestratorState.TRAINING)
                    t0 = time.perf_counter()
                    batch = self._next_batch()
                    im.train_metrics = self._train_sft(batch)
                    im.state_durations["training"] = time.perf_counter() - t0
                    im.tokens_trained = sum(len(p) for p in batch.prompt_tokens)
                    if cfg.inference_preview_enabled and cfg.max_tokens > 0 and self.infer_engine is not None:
                        # preview only, not used for the loss (src/orchestrator/colocate_orchestrator.py:459-466):
                        # one sample for the batch's first prompt from the weights just trained
                        self._set_state(OrchestratorState.INFERRING)
                        t0 = time.perf_counter()
                        im.weights_version = self._sync_weights(it)
                        out = self.infer_engine.generate(batch.prompt_tokens[:1], cfg.max_tokens, cfg.temperature, cfg.top_p)
                        im.tokens_generated = len(out[0]) if out and out[0] else 0
                        if out and out[0] and self.data is not None:
                            self.last_preview = self.data.tokenizer.decode(out[0], skip_special_tokens=True)
                            logger.info("preview: %s", ascii(self.last_preview[:120]))
                        im.state_durations["inferring"] = time.perf_counter() - t0
                else:
                    # ---- rollout (possibly prefetched while the previous iteration trained) ----------------
                    self._set_state(OrchestratorState.INFERRING)
                    t0 = time.perf_counter()
                    ro = None
                    if pending is not None:
                        ro = await pending
                        pending = None
                        stale = self.weights_version - ro.weights_version
                        if stale > cfg.async_pipeline_max_staleness:
                            logger.info("dropping a rollout that is %d versions stale", stale)
                            ro = None
                    if ro is None:
                        nb = self._next_batch()
                        ro = await self._rollout_vllm(nb) if self._uses_vllm() else self._rollout(nb)
                    im.rollout_staleness = self.weights_version - ro.weights_version
                    im.state_durations["inferring"] = time.perf_counter() - t0
                    im.tokens_generated = sum(len(r) for g in ro.responses for r in g)
                    # ---- reward ------------------------------------------------------------------------------
                    self._set_state(OrchestratorState.REWARDING)
                    t0 = time.perf_counter()
                    rewards = self._rewards(ro)
                    flat = [x for g in rewards for x in g]
                    im.avg_reward = sum(flat) / max(1, len(flat))
                    im.iteration_accuracy = sum(1 for x in flat if x >= 1.0) / max(1, len(flat))
                    im.state_durations["rewarding"] = time.perf_counter() - t0
                    # ---- train (next rollout overlaps on the worker thread) ---------------------------------
                    self._set_state(OrchestratorState.TRAINING)
                    t0 = time.perf_counter()
                    if cfg.async_pipeline_enabled and it + 1 < cfg.total_iterations:
                        nxt = self._next_batch()
                        pending = (asyncio.ensure_future(self._rollout_vllm(nxt)) if self._uses_vllm()
                                   else loop.run_in_executor(self._pool, self._rollout, nxt))
                    im.train_metrics = self._train_grpo(ro, rewards)
                    im.tokens_trained = sum(len(p) + len(r) for p, g in zip(ro.batch.prompt_tokens, ro.responses) for r in g)
                    im.state_durations["training"] = time.perf_counter() - t0
                    # ---- sleep / sync / wake -------------------------------------------------------------------
                    self._set_state(OrchestratorState.SLEEPING)
                    if self.vllm_client is not None:
                        await self.vllm_client.sleep(cfg.sleep_level)
                    self._set_state(OrchestratorState.SYNCING)
                    t0 = time.perf_counter()
                    if pending is not None and cfg.async_pipeline_max_staleness <= 0:
                        ro_next = await pending      # staleness 0: finish the rollout before weights change
                        pending = loop.create_future()
                        pending.set_result(ro_next)
                    await self._sync(it)
                    im.state_durations["syncing"] = time.perf_counter() - t0
                    if self.vllm_client is not None:
                        await self._wake_with_retries()
                im.weights_version = self.weights_version
            except Exception as e:  # noqa: BLE001 - an iteration may fail; the loop continues
                if isinstance(e, PeerLostError):
                    raise           # a rank is gone: no later iteration can complete its collectives
                await self._handle_error(it, e, im)
            im.total_time = time.perf_counter() - t_iter
            self.metrics.append(im)
            self._record(im)
            if cfg.checkpoint_save_enabled and cfg.checkpoint_save_interval > 0 and (it + 1) % cfg.checkpoint_save_interval == 0:
                self._save_checkpoint(f"iter_{it + 1}", it + 1)
            if cfg.memory_profile_interval > 0 and (it + 1) % cfg.memory_profile_interval == 0:
                self.memory.snapshot(f"iter_{it + 1}")
            if it + 1 < cfg.total_iterations and self._stop_agreed():
                # a stop was asked for (SIGTERM from a scheduler about to take the node, an operator): leave at an
                # iteration boundary, with a checkpoint that ``resume_from`` continues from
                logger.info("stop requested: leaving after iteration %d of %d", it + 1, cfg.total_iterations)
                self.stopped_early = True
                if cfg.checkpoint_save_enabled and self._last_checkpoint_path != os.path.join(
                        cfg.checkpoint_save_dir, f"iter_{it + 1}"):
                    self._save_checkpoint(f"iter_{it + 1}", it + 1)
                break
        if pending is not None:
            try:
                await pending
            except Exception:  # noqa: BLE001
                pass
        if not self.stopped_early:
            if cfg.eval_num_prompts > 0:
                self._do_eval("after")
            if cfg.checkpoint_save_enabled:
                self._save_checkpoint("final", max(self.start_iteration, cfg.total_iterations))
        self._set_state(OrchestratorState.DONE)
        self._write_final_artifacts()
        return self.metrics

    def request_stop(self):
        """Ask the loop to end at the next iteration boundary (safe to call from a signal handler or another thread).
        The run then saves ``iter_N`` (when checkpoints are enabled), skips the final evaluation and the ``final``
        checkpoint, writes its artefacts and returns; ``resume_from`` that checkpoint continues the run."""
        self._stop_requested = True

    def _stop_agreed(self) -> bool:
        """True when any rank was asked to stop: signals reach the ranks at different moments, and all of them must
        leave after the same iteration (one small all-reduce per iteration, between the iteration's own collectives)."""
        flag = self._stop_requested
        ctx = self.train_engine.parallel_ctx
        import torch.distributed as dist
        if ctx.world_size > 1 and dist.is_initialized():
            t = torch.tensor([int(flag)], dtype=torch.int32, device=self.train_engine.device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            flag = bool(int(t.item()))
        return flag

    # ---- stage methods under the reference's names (src/orchestrator/colocate_orchestrator.py:886-1060,
    # 1644-1740): its loop and its tests address the stages as _do_* coroutines --------------------------------
    async def _do_inference(self, batch: GRPOBatch, num_samples: Optional[int] = None) -> List[List[List[int]]]:
        """K sampled responses per prompt of ``batch`` as token-id lists ``[B][K][tokens]``."""
        if num_samples is not None and num_samples != self.config.num_samples_per_prompt:
            saved, self.config.num_samples_per_prompt = self.config.num_samples_per_prompt, num_samples
            try:
                return self._rollout(batch).responses
            finally:
                self.config.num_samples_per_prompt = saved
        return self._rollout(batch).responses

    async def _do_inference_async(self, batch: GRPOBatch, num_samples: Optional[int] = None):
        """The rollout on the worker thread, so that it overlaps training on the event-loop thread."""
        loop = asyncio.get_running_loop()
        return (await loop.run_in_executor(self._pool, self._rollout, batch)).responses

    async def _do_training(self, batch: GRPOBatch, responses: List[List[List[int]]], rewards: List[List[float]]) -> TrainMetrics:
        return self._train_grpo(_Rollout(batch, responses, None, self.weights_version, 0.0), rewards)

    async def _do_sft_training(self, batch: GRPOBatch) -> TrainMetrics:
        return self._train_sft(batch)

    async def _do_weight_sync(self, iteration: int = 0):
        await self._sync(iteration)

    async def _do_weight_sync_async(self, iteration: int = 0):
        await self._sync(iteration)

    async def _sync(self, iteration: int):
        if self.vllm_client is not None:
            state = self.train_engine.export_weights("cuda" if torch.cuda.is_available() else None)
            await self.ipc.push_weights(state, sleep_first=False)
            self.weights_version += 1
        else:
            self._sync_weights(iteration)

    async def _wake_with_retries(self):
        cfg = self.config
        for attempt in range(cfg.max_retries):
            try:
                await self.vllm_client.wake_up()
                return
            except Exception as e:  # noqa: BLE001
                logger.warning("wake_up attempt %d failed: %s", attempt + 1, e)
                await asyncio.sleep(cfg.retry_delay)
        raise RuntimeError("inference server did not wake up")

    async def _handle_error(self, it, e=None, im: Optional[IterationMetrics] = None):
        """``(iteration, error, metrics)``; the reference's ``(error, stage_name)`` form is accepted too
        (src/orchestrator/colocate_orchestrator.py:1742-1775).  Marks the state, records the error on the iteration and
        wakes a sleeping inference server so that the next iteration can run."""
        if isinstance(it, BaseException):
            it, e = (e if e is not None else "?"), it
        logger.error("iteration %s failed: %s: %s", it, type(e).__name__, e)
        self._set_state(OrchestratorState.ERROR)
        if im is not None:
            im.error = f"{type(e).__name__}: {e}"
        if self.vllm_client is not None:
            try:
                await self._wake_with_retries()
            except Exception:  # noqa: BLE001
                pass

    # ---- the loop over replaceable stages ----------------------------------------------------------------------
    _STAGES = ("_do_inference", "_do_training", "_do_weight_sync")

    def _stages_overridden(self) -> bool:
        """True when a subclass or the caller replaced one of the stage coroutines.  ``run`` then drives the
        iteration through them one after the other (no rollout prefetch), the way the reference's loop does
        (src/orchestrator/colocate_orchestrator.py:1290-1500); the default loop calls the native stages directly."""
        return any(name in self.__dict__ or getattr(type(self), name) is not getattr(ColocateOrchestrator, name)
                   for name in self._STAGES)

    def _stage_rewards(self, batch: GRPOBatch, responses) -> List[List[float]]:
        first = next((r for g in responses for r in g), None)
        if isinstance(first, str):                                     # text from a server or a replaced stage
            return self.reward_fn(responses, batch.ground_truths)
        return self._rewards(_Rollout(batch, responses, None, self.weights_version, 0.0))

    async def _run_staged(self) -> List[IterationMetrics]:
        cfg = self.config
        import inspect
        sync_takes_iteration = len(inspect.signature(self._do_weight_sync).parameters) > 0
        for it in range(self.start_iteration, cfg.total_iterations):
            im = IterationMetrics(it)
            t_iter = time.perf_counter()
            try:
                batch = self._next_batch()
                self._set_state(OrchestratorState.INFERRING)
                t0 = time.perf_counter()
                responses = await self._do_inference(batch)
                im.state_durations["inferring"] = time.perf_counter() - t0
                if not isinstance(next((r for g in responses for r in g), None), str):      # token ids, not text
                    im.tokens_generated = sum(len(r) for g in responses for r in g)
                    im.tokens_trained = sum(len(p) + len(r) for p, g in zip(batch.prompt_tokens, responses) for r in g)
                self._set_state(OrchestratorState.REWARDING)
                t0 = time.perf_counter()
                rewards = self._stage_rewards(batch, responses)
                flat = [x for g in rewards for x in g]
                im.avg_reward = sum(flat) / max(1, len(flat))
                im.iteration_accuracy = sum(1 for x in flat if x >= 1.0) / max(1, len(flat))
                im.state_durations["rewarding"] = time.perf_counter() - t0
                self._set_state(OrchestratorState.TRAINING)
                t0 = time.perf_counter()
                im.train_metrics = await self._do_training(batch, responses, rewards)
                im.state_durations["training"] = time.perf_counter() - t0
                self._set_state(OrchestratorState.SLEEPING)
                if self.vllm_client is not None:
                    await self.vllm_client.sleep(cfg.sleep_level)
                self._set_state(OrchestratorState.SYNCING)
                t0 = time.perf_counter()
                await (self._do_weight_sync(it) if sync_takes_iteration else self._do_weight_sync())
                im.state_durations["syncing"] = time.perf_counter() - t0
                if self.vllm_client is not None:
                    await self._wake_with_retries()
                im.weights_version = self.weights_version
            except Exception as e:  # noqa: BLE001 - an iteration may fail; the loop continues
                if isinstance(e, PeerLostError):
                    raise           # a rank is gone: no later iteration can complete its collectives
                await self._handle_error(it, e, im)
            im.total_time = time.perf_counter() - t_iter
            self.metrics.append(im)
            if self.artifacts is not None:
                self._record(im)
            else:
                im.accuracy = im.iteration_accuracy
        self._set_state(OrchestratorState.DONE)
        if self.artifacts is not None:
            self._write_final_artifacts()
        return self.metrics

    # the reference keeps these collaborators under private names (its tests and subclasses set them directly)
    _vllm_client = property(lambda self: self.vllm_client, lambda self, v: setattr(self, "vllm_client", v))
    _reward_fn = property(lambda self: self.reward_fn, lambda self, v: setattr(self, "reward_fn", v))
    _data_pipeline = property(lambda self: self.data, lambda self, v: setattr(self, "data", v))

    # ---- artefacts ------------------------------------------------------------------------------------------
    def _record(self, im: IterationMetrics):
        cum = [m.iteration_accuracy for m in self.metrics]
        im.cumulative_accuracy = sum(cum) / max(1, len(cum))
        im.accuracy = im.iteration_accuracy
        tm = im.train_metrics
        row = {"iteration": im.iteration, "total_time": im.total_time, "avg_reward": im.avg_reward,
               "accuracy": im.iteration_accuracy, "cumulative_accuracy": im.cumulative_accuracy,
               "tokens_generated": im.tokens_generated, "tokens_trained": im.tokens_trained,
               "weights_version": im.weights_version, "rollout_staleness": im.rollout_staleness, "error": im.error,
               **{f"t_{k}": v for k, v in im.state_durations.items()}}
        if tm is not None:
            row.update({"loss": tm.loss, "policy_loss": tm.policy_loss, "kl": tm.kl_divergence,
                        "grad_norm": tm.grad_norm, "lr": tm.learning_rate, "step": tm.step})
            row.update({k: v for k, v in (tm.extras or {}).items()})
        self.artifacts.append_jsonl("metrics", row)
        if self.tb is not None and tm is not None:
            self.tb.add_scalar("train/loss", tm.loss, im.iteration)
            self.tb.add_scalar("train/grad_norm", tm.grad_norm, im.iteration)
            self.tb.add_scalar("train/lr", tm.learning_rate, im.iteration)
            self.tb.add_scalar("rollout/avg_reward", im.avg_reward, im.iteration)
            self.tb.add_scalar("time/iteration_s", im.total_time, im.iteration)
        if self.compute_profiler is not None and tm is not None and (im.iteration + 1) % max(1, self.config.profile_interval) == 0:
            self.collector.record("mfu", self._mfu(im))

    def _mfu(self, im: IterationMetrics) -> float:
        cfg, mc = self.config, self.train_engine.model_config
        t = im.state_durations.get("training", 0.0)
        if t <= 0:
            return 0.0
        fl = ComputeProfiler.reference_formula_flops(mc.num_layers, self._per_rank_batch(), cfg.max_seq_len, mc.hidden_size,
                                                     mc.intermediate_size, mc.vocab_size, full=cfg.lora_rank <= 0)
        return self.compute_profiler.compute_mfu(fl / (cfg.tp_size * cfg.pp_size), t)

    def _per_rank_batch(self) -> int:
        """``training.batch_size`` is the GLOBAL batch of an iteration here: every data-parallel rank takes
        ``batch_size // dp_size`` of it.  (The reference's validator calls the key ``global_batch`` too, while its
        data path hands the full value to every rank; scale the key by ``dp_size`` when porting such a config.)"""
        return max(1, self.config.batch_size // max(1, self.config.dp_size))

    def _do_eval(self, stage: str) -> Dict:
        """Fixed-prompt evaluation before / after training (src/orchestrator/colocate_orchestrator.py:940-1060):
        SFT loss and perplexity on the reference responses, then one sampled generation per prompt scored by
        exact match, token F1 and BLEU-4.  Writes ``eval_<stage>.json`` and, after the second stage,
        ``fixed_prompt_comparison.json``.  Every rank evaluates its own data shard (ZeRO-3 needs all ranks in
        the forward); rank 0 writes."""
        cfg, eng = self.config, self.train_engine
        if cfg.eval_num_prompts <= 0 or self.data is None:
            return {}
        batch = next(iter(self.data.get_batches(cfg.eval_num_prompts)), None)
        if batch is None:
            logger.warning("no data for the %s evaluation (%d prompts wanted)", stage, cfg.eval_num_prompts)
            return {}
        tok = self.data.tokenizer
        eos = getattr(tok, "eos_token_id", None)
        references = batch.reference_responses or [str(g) for g in batch.ground_truths]
        eval_loss = perplexity = None
        if batch.reference_responses:
            resp = [list(tok.encode(t)) + ([eos] if eos is not None else []) for t in references]
            eval_loss = eng.eval_sft_loss(batch.prompt_tokens, resp)
            perplexity = math.exp(min(eval_loss, 20.0))
        samples, em = [], EvalMetrics()
        for i, (prompt, ptoks, ref) in enumerate(zip(batch.prompts, batch.prompt_tokens, references)):
            out = eng.generate(ptoks, cfg.eval_max_tokens, 0.7, 0.95, eos)
            text = tok.decode(out, skip_special_tokens=True)
            em.add(text, ref)
            samples.append({"index": i, "prompt": prompt, "generated": text, "reference": ref,
                            "generated_tokens": len(out), "exact_match": bool(compute_exact_match(text, ref)),
                            "token_f1": compute_token_f1(text, ref), "bleu4": compute_bleu4(text, ref)})
        n = max(1, len(samples))
        metrics = {"stage": stage, "step": eng.step_count, "eval_loss": eval_loss, "perplexity": perplexity,
                   "exact_match": sum(s["exact_match"] for s in samples) / n,
                   "token_f1": sum(s["token_f1"] for s in samples) / n,
                   "bleu4": sum(s["bleu4"] for s in samples) / n, "num_samples": len(samples)}
        logger.info("eval (%s): loss=%s ppl=%s exact_match=%.4f token_f1=%.4f bleu4=%.4f", stage,
                    "n/a" if eval_loss is None else f"{eval_loss:.4f}",
                    "n/a" if perplexity is None else f"{perplexity:.3f}",
                    metrics["exact_match"], metrics["token_f1"], metrics["bleu4"])
        if self.tb is not None:
            if eval_loss is not None:
                self.tb.add_scalar(f"eval/{stage}_loss", eval_loss, eng.step_count)
                self.tb.add_scalar(f"eval/{stage}_perplexity", perplexity, eng.step_count)
            self.tb.add_scalar(f"eval/{stage}_exact_match", metrics["exact_match"], eng.step_count)
            self.tb.add_scalar(f"eval/{stage}_token_f1", metrics["token_f1"], eng.step_count)
        self._eval_snapshots[stage] = samples
        self.eval_results[stage] = metrics
        self.artifacts.write_json(f"eval_{stage}.json", {"metrics": metrics, "samples": samples})
        if stage == "after" and "before" in self._eval_snapshots:
            rows = [{"index": b["index"], "prompt": b["prompt"], "reference": b["reference"],
                     "before_generated": b["generated"], "after_generated": a["generated"],
                     "before_token_f1": b["token_f1"], "after_token_f1": a["token_f1"],
                     "before_exact_match": b["exact_match"], "after_exact_match": a["exact_match"]}
                    for b, a in zip(self._eval_snapshots["before"], samples)]
            self.artifacts.write_json("fixed_prompt_comparison.json", {"samples": rows})
        return metrics

    def _save_checkpoint(self, tag: str, iterations_completed: Optional[int] = None):
        """The engine's checkpoint under ``tag`` and ``latest``, plus (rank 0) ``orchestrator_state.json``: how many
        iterations are complete, so that ``resume_from`` continues the loop and the data stream from there.  Every
        iteration draws one batch; a rollout prefetched for the next iteration is not counted (a resumed run draws
        it again)."""
        base = self.config.checkpoint_save_dir
        done = iterations_completed if iterations_completed is not None else len(self.metrics) + self.start_iteration
        for name in (tag, "latest"):
            d = os.path.join(base, name)
            self.train_engine.save_checkpoint(d)
            self._save_rollout_rng(d)
            if self.train_engine.parallel_ctx.global_rank == 0:
                self.train_engine._atomic_save({"iterations_completed": done, "batches_consumed": done,
                                                "weights_version": self.weights_version},
                                               os.path.join(d, "orchestrator_state.json"), as_json=True)
        self.train_engine.parallel_ctx.barrier()
        self._last_checkpoint_path = os.path.join(base, tag)
        self._prune_checkpoints(base)

    def _prune_checkpoints(self, base: str):
        """``checkpoint.keep_last = N`` keeps the newest N ``iter_*`` directories (by iteration number) and deletes the
        older ones, on rank 0, after the new checkpoint is complete; ``latest`` and ``final`` are never touched, nor
        anything that is not an ``iter_<number>`` directory."""
        keep = self.config.checkpoint_keep_last
        if keep <= 0 or self.train_engine.parallel_ctx.global_rank != 0:
            return
        import re
        import shutil
        found = sorted((int(m.group(1)), name) for name in os.listdir(base)
                       for m in [re.fullmatch(r"iter_(\d+)", name)] if m and os.path.isdir(os.path.join(base, name)))
        for _, name in found[:-keep]:
            shutil.rmtree(os.path.join(base, name), ignore_errors=True)

    @property
    def metrics_history(self) -> List[IterationMetrics]:
        """The per-iteration records under the reference's attribute name."""
        return self.metrics

    async def _transition(self, new_state: OrchestratorState):
        """State change as a coroutine (the reference's loop awaits its transitions)."""
        self._set_state(new_state)

    def get_summary(self) -> Dict:
        if not self.metrics:
            return {"status": "no_data"}
        ok = [m for m in self.metrics if m.error is None]
        losses = [m.train_metrics.loss for m in ok if m.train_metrics is not None]
        stage: Dict[str, float] = {}
        for m in ok:
            for k, v in m.state_durations.items():
                stage[k] = stage.get(k, 0.0) + v
        n = max(1, len(ok))
        summary = {
            "config": config_snapshot(self.config),
            "results": {"iterations": len(self.metrics), "failed_iterations": len(self.metrics) - len(ok),
                        "final_loss": losses[-1] if losses else None, "initial_loss": losses[0] if losses else None,
                        "avg_reward": sum(m.avg_reward for m in ok) / n,
                        "avg_iteration_time": sum(m.total_time for m in ok) / n,
                        "final_weights_version": self.weights_version,
                        # the reference's key names (src/orchestrator/colocate_orchestrator.py:1808-1815)
                        "completed_iterations": len(self.metrics),
                        "final_accuracy": self.metrics[-1].accuracy, "final_avg_reward": self.metrics[-1].avg_reward,
                        "best_accuracy": max(m.accuracy for m in self.metrics),
                        "avg_iteration_time_s": sum(m.total_time for m in self.metrics) / len(self.metrics),
                        "total_time_s": sum(m.total_time for m in self.metrics)},
            "stage_averages": {k: v / n for k, v in stage.items()},
            "stage_avg_durations": {k: v / n for k, v in stage.items()},
            "memory": {"peak_mb": self.memory.peak_memory_mb},
            "metrics_summary": self.collector.get_summary(),
            "system": {"world_size": self.train_engine.parallel_ctx.world_size if self.train_engine else 1,
                       "device": torch.cuda.get_device_name(0) if torch.cuda.is_available() else "cpu",
                       "wall_time_s": time.time() - self._start_time if self._start_time else 0.0},
            "performance": {"tokens_trained": sum(m.tokens_trained for m in ok),
                            "tokens_generated": sum(m.tokens_generated for m in ok),
                            "mfu_samples": self.collector.series.get("mfu", [])},
            "metrics": self.collector.summary(),
            "eval": self.eval_results,
            "state_log_tail": self.state_log[-16:],
        }
        if self.infer_engine is not None:
            summary["inference"] = self.infer_engine.get_stats()
        if self.swift is not None:
            summary["swift_sync"] = self.swift.get_stats()
        if self.weight_sync is not None:
            summary["weight_sync"] = self.weight_sync.get_stats()
        return summary

    def _performance_block(self) -> Dict:
        """Throughput and MFU of the run (src/orchestrator/colocate_orchestrator.py:1145-1280).  Two MFU
        figures: the reference's formula (no attention S^2 term, ``4H^2`` projections; kept for comparison
        with its published numbers) and exact matmul FLOPs; both against the measured sustained bf16 GEMM
        throughput of the device instead of a datasheet peak."""
        cfg, eng = self.config, self.train_engine
        mc = eng.model_config
        ok = [m for m in self.metrics if m.error is None]
        times = [m.state_durations.get("training", m.total_time) for m in ok]
        if not times or sum(times) <= 0:
            return {}
        step = sum(times) / len(times)
        full = cfg.lora_rank <= 0
        tp, pp, dp = max(1, cfg.tp_size), max(1, cfg.pp_size), max(1, cfg.dp_size)
        prof = self.compute_profiler or ComputeProfiler()
        per_rank = self._per_rank_batch()
        ref_fl = ComputeProfiler.reference_formula_flops(mc.num_layers, per_rank, cfg.max_seq_len, mc.hidden_size,
                                                         mc.intermediate_size, mc.vocab_size, full=full) / (tp * pp)
        exact_fl = ComputeProfiler.exact_flops(mc, per_rank, cfg.max_seq_len, full=full,
                                               grad_checkpoint=cfg.use_gradient_checkpoint) / (tp * pp)
        gbs = per_rank * dp
        return {
            "mfu_percent": round(100 * prof.compute_mfu(ref_fl, step), 2),
            "mfu_exact_percent": round(100 * prof.compute_mfu(exact_fl, step), 2),
            "per_gpu_training_flops": int(ref_fl), "per_gpu_training_flops_exact": int(exact_fl),
            "actual_tflops_per_gpu": round(ref_fl / step / 1e12, 2), "device_peak_tflops": prof.peak_tflops,
            "world_size": tp * pp * dp, "tp_size": tp, "pp_size": pp, "dp_size": dp, "global_batch_size": gbs,
            "tokens_per_second": round(gbs * cfg.max_seq_len / step), "samples_per_second": round(gbs / step, 2),
            "avg_step_time_s": round(step, 4), "model_params": mc.num_params(),
            "model_arch": {"num_layers": mc.num_layers, "hidden_size": mc.hidden_size,
                           "intermediate_size": mc.intermediate_size, "vocab_size": mc.vocab_size,
                           "seq_len": cfg.max_seq_len},
            "primary_metric": "mfu" if full else "tokens_per_second",
            "note": (f"MFU = forward FLOPs x {3 if full else 2} / (tp x pp) / (step time x peak); peak = measured "
                     f"sustained bf16 GEMM throughput of this device class ({prof.peak_tflops:.0f} TFLOP/s); tokens/s "
                     f"assumes {per_rank} sequences x max_seq_len tokens per rank and step (padding counted, as the "
                     f"reference does); training.batch_size is the global batch"),
        }

    def _write_final_artifacts(self):
        summary = self.get_summary()
        cfg = self.config
        summary["status"] = "completed" if self.metrics else "no_data"
        summary["mode"] = cfg.training_mode
        summary["run"] = {"started_at_unix": self._start_time, "ended_at_unix": time.time(), "output_dir": cfg.output_dir,
                          "resume_from": cfg.resume_from, "last_checkpoint_path": self._last_checkpoint_path}
        names = ["config_snapshot.json", "run_summary.json", "loss_curve.csv", "loss_curve.png", "eval_before.json",
                 "eval_after.json", "fixed_prompt_comparison.json", "memory_report.json", "tensorboard"]
        summary["artifacts"] = {n.split(".")[0]: self.artifacts.path(n) for n in names}
        summary["artifacts"]["metrics_jsonl"] = self.artifacts.path(f"metrics_rank{self.artifacts.rank}.jsonl")
        try:
            summary.setdefault("performance", {}).update(self._performance_block())
        except Exception as e:  # noqa: BLE001 - the summary is written regardless
            logger.warning("performance block not computed: %s", e)
        self.artifacts.write_json("run_summary.json", summary)
        if self.artifacts.is_main:
            with open(self.artifacts.path("loss_curve.csv"), "w", newline="") as f:
                w = csv.writer(f)
                w.writerow(["iteration", "loss", "grad_norm", "avg_reward"])
                for m in self.metrics:
                    if m.train_metrics is not None:
                        w.writerow([m.iteration, m.train_metrics.loss, m.train_metrics.grad_norm, m.avg_reward])
            self._render_loss_curve()
        self.artifacts.write_json("memory_timeline.json", self.memory.timeline(), all_ranks=True)
        rep = self.train_engine.generate_memory_report(self._per_rank_batch() * self.config.max_seq_len)
        self.artifacts.write_json("memory_report.json", rep.to_dict())
        if self.tb is not None:
            self.tb.flush()

    def _render_loss_curve(self):
        """``loss_curve.png`` next to the CSV when matplotlib is importable (the CSV is always written)."""
        rows = [(m.iteration, m.train_metrics.loss) for m in self.metrics if m.train_metrics is not None]
        if not rows:
            return
        try:
            import matplotlib
            matplotlib.use("Agg")
            import matplotlib.pyplot as plt
        except Exception:  # noqa: BLE001 - optional dependency
            logger.info("matplotlib is not installed: loss_curve.png skipped, loss_curve.csv written")
            return
        plt.figure(figsize=(8, 4.5))
        plt.plot([r[0] for r in rows], [r[1] for r in rows], marker="o", linewidth=1.5)
        plt.xlabel("Iteration")
        plt.ylabel("Loss")
        plt.title("Training loss")
        plt.grid(True, alpha=0.3)
        plt.tight_layout()
        plt.savefig(self.artifacts.path("loss_curve.png"), dpi=160)
        plt.close()

    async def shutdown(self):
        self._pool.shutdown(wait=True)
        if self.vllm_client is not None:
            await self.vllm_client.close()
        if self.tb is not None:
            self.tb.close()


class _LoRAWorker:
    """SwiftSync's view of the in-process rollout engine.

    The engine holds plain merged weights ``W_base + s * B A``.  A sync does not re-export the model: for every
    adapted projection one low-rank GEMM updates the engine's weight rows in place,

    * delta:  ``W += (s B_new) A_new + (-s B_old) A_old``   (ONE GEMM per adapted module: the new and old adapters of
      all its sub-projections stacked along the contraction, accumulate epilogue), where ``new = old + delta`` and
      ``old`` is this worker's record of what the engine currently carries;
    * full:   ``W  = W_base + s B_new A_new``                    (the trainer's frozen base as the residual operand),
      which also wipes the bf16 rounding the in-place deltas have accumulated.

    Same role as the reference's delta application on the worker (src/transfer/swift_sync.py:181-292), which adds
    the adapter deltas into a worker-side LoRA copy and re-merges.  Under tensor parallelism the trainer holds
    shards of the base, so the worker falls back to a gathered export."""

    def __init__(self, orch: ColocateOrchestrator):
        self.orch = orch
        self.applied: Optional[Dict[str, torch.Tensor]] = None      # adapter state the engine's weights carry
        self._plan = None
        self.lowrank_on_cpu = False      # tests: run the low-rank path (through the ops' CPU forms) without a GPU

    def _engine_weight(self, mod_name: str) -> torch.Tensor:
        """The engine model's weight of the module that trainer module ``mod_name`` maps to."""
        m = self.orch.infer_engine.model
        for part in mod_name.split("."):
            m = getattr(m, part) if not part.isdigit() else m[int(part)]
        return m.weight

    def _build_plan(self, eng):
        """Layout of a sync, built once.

        * ``flat``: one fp32 image of all adapter tensors (A and B of every adapted projection, in the key order of
          the payload) with a scale vector (1 on A entries, alpha/r on B entries).
        * ``cat``: one bf16 buffer holding, per adapted MODULE (a fused q|k|v or gate|up layer carries several
          adapters), the stacked operands ``Bcat [N, 2R]`` and ``Acat [2R, K]``: columns / rows ``[0, R)`` take the new
          adapters (each B in its own row range and rank columns: block diagonal), ``[R, 2R)`` the old ones, so that
          ``W += Bcat Acat`` is ``W += sum_i s B_i,new A_i,new - s B_i,old A_i,old`` in ONE GEMM per module.  The
          zero blocks are never written.  ``dst_new`` / ``dst_old`` map every entry of ``flat`` to its place in
          ``cat``: a sync fills ``cat`` with two bulk index copies, whatever the number of adapters."""
        from ..model.lora import LinearWithLoRA
        dev, dt = eng.device, eng.dtype
        keys, shapes, offs, scale, n = [], [], [], [], 0
        dst_new, dst_old, sign_old, mods, cat_n = [], [], [], [], 0
        for name, mod in eng.model.named_modules():
            if not isinstance(mod, LinearWithLoRA) or not mod.adapters:
                continue
            N, K = mod.base.weight.shape
            order = sorted(mod.ranges.items(), key=lambda kv: kv[1][0])
            R = sum(mod.adapters[t].rank for t, _ in order)
            b_off, a_off = cat_n, cat_n + N * 2 * R
            cat_n = a_off + 2 * R * K
            r0 = 0
            for tgt, (s0, e0) in order:
                ad = mod.adapters[tgt]
                r = ad.rank
                for leaf, t, sc in (("lora_A", ad.lora_A, 1.0), ("lora_B", ad.lora_B, float(ad.scaling))):
                    keys.append(f"{name}.{tgt}.{leaf}")
                    shapes.append(tuple(t.shape))
                    offs.append(n)
                    scale.append(torch.full((t.numel(),), sc, dtype=torch.float32))
                    n += t.numel()
                    if leaf == "lora_A":        # [r, K] -> rows r0.. of Acat (new), rows R + r0.. (old)
                        i = torch.arange(r)[:, None] * K + torch.arange(K)[None, :]
                        dst_new.append((a_off + r0 * K + i).reshape(-1))
                        dst_old.append((a_off + (R + r0) * K + i).reshape(-1))
                        sign_old.append(torch.ones(t.numel()))
                    else:                       # [e0 - s0, r] -> rows s0.. of Bcat, columns r0.. (new) / R + r0.. (old)
                        i = (s0 + torch.arange(e0 - s0))[:, None] * (2 * R) + torch.arange(r)[None, :]
                        dst_new.append((b_off + r0 + i).reshape(-1))
                        dst_old.append((b_off + R + r0 + i).reshape(-1))
                        sign_old.append(-torch.ones(t.numel()))
                r0 += r
            mods.append((name, N, K, R, b_off, a_off, mod.base.weight))
        cat = torch.zeros(cat_n, dtype=dt, device=dev)
        jobs = []
        for name, N, K, R, b_off, a_off, base_w in mods:
            bcat = cat[b_off:b_off + N * 2 * R].view(N, 2 * R)
            acat = cat[a_off:a_off + 2 * R * K].view(2 * R, K)
            jobs.append((bcat, acat, bcat[:, :R], acat[:R], self._engine_weight(name), base_w))
        sc = torch.cat(scale).to(dev)
        from ..sync.double_buffer import FlatLayout
        self._plan = {"keys": keys, "shapes": shapes, "offs": offs, "numel": n, "jobs": jobs, "scale": sc,
                      "layout": FlatLayout(keys, shapes),
                      "scale_old": sc * torch.cat(sign_old).to(dev), "cat": cat,
                      "dst_new": torch.cat(dst_new).to(dev), "dst_old": torch.cat(dst_old).to(dev),
                      "flat": torch.zeros(n, dtype=torch.float32, device=dev)}
        return self._plan

    @torch.no_grad()
    def update_weights(self, state, mode: str = "full"):
        from .. import ops
        orch = self.orch
        eng = orch.train_engine
        if eng.parallel_ctx.tp_size > 1 or (eng.device.type != "cuda" and not self.lowrank_on_cpu):
            merged = orch._merged_clone()
            from ..model.hf_io import hf_named_tensors
            orch.infer_engine.load_weights(dict(hf_named_tensors(merged)))
            return
        plan = self._plan or self._build_plan(eng)
        dev, dt = eng.device, eng.dtype
        if any(k not in state for k in plan["keys"]):
            raise KeyError("SwiftSync payload does not cover every adapter tensor of the model")
        from ..sync.double_buffer import FlatState
        if isinstance(state, FlatState) and state.layout.keys == tuple(plan["keys"]):
            incoming = state.flat.to(dev, torch.float32)          # already one tensor in the plan's order
        else:
            incoming = torch.cat([state[k].reshape(-1) for k in plan["keys"]]).to(dev, torch.float32)
        old, cat = plan["flat"], plan["cat"]
        delta = mode == "delta" and self.applied is not None
        new = old + incoming if delta else incoming
        cat.index_copy_(0, plan["dst_new"], (new * plan["scale"]).to(dt))          # A_new and s * B_new
        if delta:
            cat.index_copy_(0, plan["dst_old"], (old * plan["scale_old"]).to(dt))   # A_old and -s * B_old
        with orch.infer_engine.paused():        # a rollout on the worker thread waits at its next step boundary
            for bcat, acat, b_new, a_new, w, base_w in plan["jobs"]:
                if delta:
                    # W += [s B_new | -s B_old] [A_new ; A_old]: one accumulate GEMM of contraction length 2R per module
                    ops.gemm(bcat, acat, b_mn=True, out=w, accumulate=True)
                else:
                    ops.gemm(b_new, a_new, b_mn=True, out=w, residual=base_w)
            plan["flat"] = new
            self.applied = FlatState(plan["layout"], new)       # name -> view of the image, made when asked for
            orch.infer_engine.on_weights_updated()
