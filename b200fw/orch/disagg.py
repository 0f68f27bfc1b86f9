"""Disaggregated orchestrator: trainer ranks and rollout ranks are two groups of ONE torchrun world
(e.g. GPUs 0-3 train with ZeRO-2, GPUs 4-7 run the native engine), instead of the reference's Ray
placement group with ``TrainWorker`` / ``InferWorker`` actors and object-store transfers
(src/orchestrator/disagg_orchestrator.py:88-500).

Per iteration: every rollout rank generates for its share of the prompts while the trainer ranks train
on the previous iteration's samples (pipeline mode; ``sequential`` runs the two phases one after the
other), the samples travel trainer-ward as token tensors, and the weights travel engine-ward through
the weight-transfer manager (peer write over NVLink, or the NCCL broadcast baseline).  The overlap
ratio reported is ``min(train, rollout) / max(train, rollout)`` of the concurrent phases.
"""
from __future__ import annotations

import time
from dataclasses import dataclass
from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from ..obs import get_logger

logger = get_logger("orch.disagg")


@dataclass
class DisaggConfig:
    model_path: str = ""
    model_preset: Optional[str] = None
    num_train_gpus: int = 4
    num_infer_gpus: int = 4
    train_zero_stage: int = 2
    total_iterations: int = 10
    batch_size: int = 64                 # prompts per iteration (global)
    num_samples_per_prompt: int = 8
    prompt_len: int = 256
    max_tokens: int = 512
    temperature: float = 0.8
    top_p: float = 0.95
    learning_rate: float = 1e-5
    lora_rank: int = 0
    grpo_beta: float = 0.01
    grpo_clip_eps: float = 0.2
    gradient_accumulation_steps: int = 1
    mode: str = "pipeline"               # "pipeline" | "sequential"
    transfer_backend: str = "nccl"       # "peer_write" | "nccl"
    max_staleness: int = 1
    kv_cache_dtype: str = "fp16"
    kv_num_blocks: int = 0               # 0: sized for one iteration's rollouts of this rank (+10 %)
    c3po_plus_enabled: bool = True       # train in token-budgeted chunks instead of one B*K-sequence forward
    c3po_plus_token_budget: int = 256
    c3po_plus_target_batch_tokens: int = 16384
    seed: int = 0
    synthetic_reward_dense_weight: float = 0.5   # dense shaping term of the synthetic rule reward: a random-init policy
                                                 # never earns the sparse reward, and all-zero advantages train nothing
    output_dir: str = "outputs_disagg"
    backend: Optional[str] = None        # process-group backend (default by device)
    # ---- accepted for configs written against the reference (src/orchestrator/disagg_orchestrator.py:39-70) ----
    use_flash_attn: bool = True          # every attention_backend value runs the native flash kernel
    attention_backend: str = "flash_attn"
    inference_backend: str = "custom"    # rollout ranks run the native engine; a vLLM server is not driven from here
    async_weight_update: bool = True
    max_data_samples: int = 0
    heartbeat_interval_s: float = 0.0    # > 0: ranks watch each other over the rendezvous store; an iteration is not
    heartbeat_timeout_s: float = 10.0    # started once a peer is gone (PeerLostError instead of a hung collective)

    # The reference sizes its two groups by tensor-parallel degree and GPU lists and names the sync backend and the
    # overlap switch differently (src/orchestrator/disagg_orchestrator.py:40-70; its run_disaggregated.py passes
    # these as keywords).  Given, they set the fields above; afterwards they always mirror them.
    train_tp_size: Optional[int] = None
    infer_tp_size: Optional[int] = None
    train_gpus: Optional[List[int]] = None
    infer_gpus: Optional[List[int]] = None
    weight_sync_backend: Optional[str] = None           # "nccl" | "peer_write"; "ray_object_store" runs as "nccl" here
    overlap_training_inference: Optional[bool] = None

    def __post_init__(self):
        if self.train_gpus is not None:
            self.num_train_gpus = len(self.train_gpus)
        elif self.train_tp_size is not None:
            self.num_train_gpus = int(self.train_tp_size)
        if self.infer_gpus is not None:
            self.num_infer_gpus = len(self.infer_gpus)
        elif self.infer_tp_size is not None:
            self.num_infer_gpus = int(self.infer_tp_size)
        if self.weight_sync_backend is not None:
            self.transfer_backend = self.weight_sync_backend if self.weight_sync_backend in ("nccl", "peer_write") else "nccl"
        if self.overlap_training_inference is not None:
            self.mode = "pipeline" if self.overlap_training_inference else "sequential"
        self.train_tp_size, self.infer_tp_size = self.num_train_gpus, self.num_infer_gpus
        self.train_gpus = list(range(self.num_train_gpus))
        self.infer_gpus = list(range(self.num_train_gpus, self.num_train_gpus + self.num_infer_gpus))
        self.weight_sync_backend = self.transfer_backend
        self.overlap_training_inference = self.mode == "pipeline"


@dataclass
class DisaggIterationMetrics:
    iteration: int
    train_time: float = 0.0
    rollout_time: float = 0.0
    sync_time: float = 0.0
    total_time: float = 0.0
    overlap_ratio: float = 0.0
    loss: float = 0.0
    avg_reward: float = 0.0
    weights_version: int = 0
    accuracy: float = 0.0
    train_metrics: Optional[object] = None       # TrainMetrics of the iteration's last optimizer step (trainer ranks)

    # the reference's field names (src/orchestrator/disagg_orchestrator.py:73-85)
    @property
    def infer_time(self) -> float:
        return self.rollout_time

    @property
    def weight_version(self) -> int:
        return self.weights_version


class _PromptBatch(list):
    """Prompt token lists of one iteration with their ground truths attached."""
    truths: Optional[List] = None


class DisaggOrchestrator:
    """Run the same object on every rank of the world; the rank decides its role."""

    def __init__(self, config: DisaggConfig, train_engine_factory=None, infer_engine_factory=None, reward_fn=None,
                 data=None):
        self.config = config
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        self.world = dist.get_world_size() if dist.is_initialized() else 1
        self.is_trainer = self.rank < config.num_train_gpus
        self.train_engine = None
        self.infer_engine = None
        self.train_group = self.infer_group = None
        self.train_engine_factory, self.infer_engine_factory = train_engine_factory, infer_engine_factory
        self.reward_fn = reward_fn
        self.data, self._batches = data, None       # optional GSM8KDataPipeline-style source (dp_rank 0 of 1 everywhere)
        self.metrics: List[DisaggIterationMetrics] = []
        self.weights_version = 0
        self.transfer = None

    # ---- set-up ----------------------------------------------------------------------------------------------
    def initialize(self):
        cfg = self.config
        assert cfg.num_train_gpus + cfg.num_infer_gpus == self.world, "train + infer GPUs must equal WORLD_SIZE"
        self.heartbeat = None
        if cfg.heartbeat_interval_s > 0:
            from ..dist.heartbeat import RankHeartbeat
            self.heartbeat = RankHeartbeat.from_default_group(cfg.heartbeat_interval_s, cfg.heartbeat_timeout_s)
            if self.heartbeat is not None:
                self.heartbeat.start()
        tr = list(range(cfg.num_train_gpus))
        inf = list(range(cfg.num_train_gpus, self.world))
        self.train_group = dist.new_group(tr)
        self.infer_group = dist.new_group(inf)
        # one sync group per trainer-leader -> all engines (leader = rank 0)
        self.sync_group = dist.new_group([0] + inf)
        if self.is_trainer:
            self.train_engine = self.train_engine_factory(self.train_group, len(tr), self.rank)
        else:
            self.infer_engine = self.infer_engine_factory(self.rank - cfg.num_train_gpus)
        from ..sync import WeightTransferManager
        want_peer = cfg.transfer_backend == "peer_write"
        if want_peer and not torch.cuda.is_available():
            logger.warning("transfer_backend=peer_write needs CUDA peer memory; using the collective broadcast")
            want_peer = False
        # every trainer rank takes part in the export (TP / ZeRO-3 gathers); rank 0 needs the tensor layout
        layout_state = self.train_engine.export_weights() if (want_peer and self.is_trainer) else None
        if self.rank == 0 or not self.is_trainer:
            if want_peer:
                # cast + checksum kernel writes straight into every engine's staging buffer over NVLink; the buffers
                # are symmetric memory of the (trainer leader + engines) group, so all its members build it together
                from ..model.hf_io import hf_named_tensors
                from ..sync import PeerWeightSync
                if self.is_trainer:
                    layout = [(k, tuple(v.shape)) for k, v in layout_state.items()]
                    dtype = next(iter(layout_state.values())).dtype
                else:
                    layout = [(k, tuple(v.shape)) for k, v in hf_named_tensors(self.infer_engine.model)]
                    dtype = next(self.infer_engine.model.parameters()).dtype
                peer = PeerWeightSync(layout, dtype, group=self.sync_group, sender_rank=0)
                self.transfer = WeightTransferManager("peer_write", peer_sync=peer)
            else:
                self.transfer = WeightTransferManager("nccl", self.sync_group, src_rank=0)
        if self.data is not None:
            # every rank reads the same pipeline, so every rank refuses the same mismatch here, once, with the reason
            tok = self.data.tokenizer
            try:
                tok_vocab = len(tok)
            except TypeError:
                tok_vocab = int(getattr(tok, "vocab_size", 0) or 0)
            vocab = (self.train_engine.model_config.vocab_size if self.is_trainer else self.infer_engine.config.vocab_size)
            if tok_vocab > vocab:
                raise ValueError(f"the tokenizer has {tok_vocab} ids but the model's vocabulary is {vocab}: its prompts "
                                 "cannot be embedded (wrong model / tokenizer pair)")
        if self.reward_fn is None and self.data is not None:
            from ..reward import GSM8KRewardFunction
            self.reward_fn = GSM8KRewardFunction()
        if self.reward_fn is None:
            from ..reward import SyntheticTokenReward
            vocab = (self.train_engine.model_config.vocab_size if self.is_trainer else self.infer_engine.config.vocab_size)
            self.reward_fn = SyntheticTokenReward(vocab, cfg.seed, dense_weight=cfg.synthetic_reward_dense_weight)
        return self

    # ---- phases ------------------------------------------------------------------------------------------------
    def _prompts(self, iteration: int) -> List[List[int]]:
        """This iteration's prompts, identical on every rank (no transfer needed for them): the next batch of the
        data pipeline when one was given (every rank reads the same un-sharded pipeline; the ground truths ride
        along on the returned list for the reward), else seeded random tokens."""
        if self.data is not None:
            if self._batches is None:
                self._batches = self.data.get_batches(self.config.batch_size)
            try:
                b = next(self._batches)
            except StopIteration:
                self._batches = self.data.get_batches(self.config.batch_size)
                b = next(self._batches)
            out = _PromptBatch(b.prompt_tokens)
            out.truths = list(b.ground_truths)
            return out
        import random
        rng = random.Random(self.config.seed * 7919 + iteration)
        vocab = (self.train_engine.model_config.vocab_size if self.is_trainer else self.infer_engine.config.vocab_size)
        return [[rng.randrange(3, vocab) for _ in range(self.config.prompt_len)] for _ in range(self.config.batch_size)]

    def _rollout_share(self, prompts: List[List[int]]):
        cfg = self.config
        i = self.rank - cfg.num_train_gpus
        mine = list(range(i, len(prompts), cfg.num_infer_gpus))
        reqs = [prompts[j] for j in mine for _ in range(cfg.num_samples_per_prompt)]
        outs = self.infer_engine.generate(reqs, cfg.max_tokens, cfg.temperature, cfg.top_p)
        K = cfg.num_samples_per_prompt
        return {j: [o or [0] for o in outs[n * K:(n + 1) * K]] for n, j in enumerate(mine)}

    def _exchange_samples(self, local: Optional[Dict[int, List[List[int]]]],
                          error: Optional[str] = None) -> Dict[int, List[List[int]]]:
        """Rollout ranks publish their samples; everyone ends up with the full set (token id lists).  A rank whose
        phase failed publishes the error instead, and every rank raises it here, together: nobody is left waiting in
        a later collective for a rank that has gone."""
        box = [None] * self.world
        dist.all_gather_object(box, {"samples": local or {}, "error": error})
        failed = [(r, d["error"]) for r, d in enumerate(box) if d["error"]]
        if failed:
            raise RuntimeError("; ".join(f"rank {r} failed before the sample exchange: {e}" for r, e in failed))
        merged: Dict[int, List[List[int]]] = {}
        for d in box:
            merged.update(d["samples"])
        return merged

    def _train(self, prompts, samples) -> float:
        cfg = self.config
        n_tr = cfg.num_train_gpus
        mine = list(range(self.rank, len(prompts), n_tr))
        P = [prompts[j] for j in mine]
        R = [samples[j] for j in mine]
        truths = getattr(prompts, "truths", None)
        if truths is not None:      # text rule reward: decode the sampled ids, score against the ground truths
            tok = self.data.tokenizer
            rewards = self.reward_fn([[tok.decode(r, skip_special_tokens=True) for r in g] for g in R],
                                     [truths[j] for j in mine])
        else:
            rewards = self.reward_fn(R, mine)
        eng = self.train_engine
        if cfg.c3po_plus_enabled:
            from ..train.c3po import C3POConfig, C3POPlusScheduler
            from ..train.engine import TrainEngine
            sched = C3POPlusScheduler(C3POConfig(True, cfg.c3po_plus_token_budget, cfg.c3po_plus_target_batch_tokens))
            adv = [TrainEngine.group_advantages(r) for r in rewards]
            subs = sched.split_and_pack(P, R, rewards, adv)
            m = None
            for i, sb in enumerate(subs):
                last = i == len(subs) - 1
                m = eng.grpo_step(**sb, skip_optimizer_step=not last, reset_behavior_baseline=True, close_window=last)
        else:
            m = eng.grpo_step(P, R, rewards)
        self._last_reward = sum(x for g in rewards for x in g) / max(1, sum(len(g) for g in rewards))
        return m.loss

    def _sync_weights(self):
        t0 = time.perf_counter()
        if self.is_trainer:
            state = self.train_engine.export_weights()        # collective over the trainer group (ZeRO-3 gathers)
            if self.rank == 0:
                self.transfer.sync_weights(True, state)
        else:
            from ..model.hf_io import hf_named_tensors
            templates = dict(hf_named_tensors(self.infer_engine.model))
            self.transfer.sync_weights(False, engine=self.infer_engine, templates=templates)
        self.weights_version += 1
        return time.perf_counter() - t0

    # ---- loop ----------------------------------------------------------------------------------------------------
    def run(self) -> List[DisaggIterationMetrics]:
        cfg = self.config
        prev = None     # (prompts, samples) generated in the previous iteration, trained in this one
        for it in range(cfg.total_iterations + (1 if cfg.mode == "pipeline" else 0)):
            if getattr(self, "heartbeat", None) is not None:
                self.heartbeat.check()           # a peer is gone: do not walk into this iteration's collectives
            t_iter = time.perf_counter()
            m = DisaggIterationMetrics(it)
            prompts = self._prompts(it)
            do_rollout = it < cfg.total_iterations
            # wall-clock spans of this rank's phases (same node: time.time() is comparable across the processes)
            span_train, span_roll = [float("inf"), float("-inf")], [float("inf"), float("-inf")]
            t0 = time.perf_counter()
            w0 = time.time()
            local, failure = None, None
            try:
                local = self._rollout_share(prompts) if (not self.is_trainer and do_rollout) else None
            except Exception as e:  # noqa: BLE001 - carried to every rank by the sample exchange
                logger.error("rollout failed on rank %d: %r", self.rank, e)
                failure = f"{type(e).__name__}: {e}"
            if not self.is_trainer:
                m.rollout_time = time.perf_counter() - t0
                if do_rollout:
                    span_roll = [w0, time.time()]
            if cfg.mode == "pipeline":
                if self.is_trainer and prev is not None:
                    t1 = time.perf_counter()
                    w1 = time.time()
                    m.loss = self._train(*prev)
                    m.train_time = time.perf_counter() - t1
                    span_train = [w1, time.time()]
                samples = self._exchange_samples(local, failure)
                prev = (prompts, samples) if do_rollout else None
            else:
                samples = self._exchange_samples(local, failure)
                if self.is_trainer:
                    t1 = time.perf_counter()
                    w1 = time.time()
                    m.loss = self._train(prompts, samples)
                    m.train_time = time.perf_counter() - t1
                    span_train = [w1, time.time()]
            m.sync_time = self._sync_weights()
            m.total_time = time.perf_counter() - t_iter
            times = torch.tensor([m.train_time, m.rollout_time], dtype=torch.float64)
            if torch.cuda.is_available() and dist.get_backend() == "nccl":
                times = times.cuda()
            dist.all_reduce(times, op=dist.ReduceOp.MAX)
            m.train_time, m.rollout_time = float(times[0]), float(times[1])
            # measured overlap: the training phase spans [earliest trainer start, latest trainer end], the rollout
            # phase likewise; the ratio is the time both were running over the shorter phase (1 = fully hidden)
            lo = torch.tensor([span_train[0], span_roll[0]], dtype=torch.float64)
            hi = torch.tensor([span_train[1], span_roll[1]], dtype=torch.float64)
            if times.is_cuda:
                lo, hi = lo.cuda(), hi.cuda()
            dist.all_reduce(lo, op=dist.ReduceOp.MIN)
            dist.all_reduce(hi, op=dist.ReduceOp.MAX)
            lo, hi = lo.tolist(), hi.tolist()
            m.overlap_ratio = 0.0
            if all(map(lambda v: v not in (float("inf"), float("-inf")), lo + hi)):
                both = min(hi[0], hi[1]) - max(lo[0], lo[1])
                shorter = min(hi[0] - lo[0], hi[1] - lo[1])
                m.overlap_ratio = max(0.0, both) / shorter if shorter > 0 else 0.0
            m.avg_reward = getattr(self, "_last_reward", 0.0)
            m.weights_version = self.weights_version
            self.metrics.append(m)
        return self.metrics

    def get_summary(self) -> Dict:
        n = max(1, len(self.metrics))
        return {"iterations": len(self.metrics), "role": "trainer" if self.is_trainer else "rollout",
                "avg_iteration_s": sum(m.total_time for m in self.metrics) / n,
                "avg_train_s": sum(m.train_time for m in self.metrics) / n,
                "avg_rollout_s": sum(m.rollout_time for m in self.metrics) / n,
                "avg_sync_s": sum(m.sync_time for m in self.metrics) / n,
                "avg_overlap_ratio": sum(m.overlap_ratio for m in self.metrics) / n,
                "final_loss": self.metrics[-1].loss if self.metrics else None,
                "weights_version": self.weights_version}

    def shutdown(self):
        hb = getattr(self, "heartbeat", None)
        if hb is not None:
            hb.announce_leave("shutdown")
