"""TrainEngine: SFT and GRPO steps over the parallel Qwen3 model.

Public surface of the reference engine (src/engines/train_engine.py:53-1768): ``TrainConfig`` /
``TrainMetrics`` with the same fields, ``initialize``, ``sft_step``, ``grpo_step``, ``generate``,
``eval_sft_loss``, ``export_weights``, ``export_lora_delta``, ``save_checkpoint``, ``load_checkpoint``,
``generate_memory_report``.  Differences by design: losses never materialise ``[B,S,V]`` logits,
gradient norm / clip / NaN guard / AdamW run on the device inside the optimizer, batches reach the
GPU from pinned host buffers, and full-SFT checkpoints include the base weights.
"""
from __future__ import annotations

import copy
import json
import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from ..dist.context import ParallelContext
from ..model import (ModelConfig, PRESETS, ParallelTransformerModel, apply_lora, get_lora_state_dict,
                     load_from_hf_checkpoint, merge_lora_weights, read_hf_config, save_hf_checkpoint)
from ..model.lora import LinearWithLoRA, load_lora_state_dict
from ..obs.logging import get_logger
from ..obs.memory import MemoryBreakdown, MemoryProfiler, MemoryReport
from ..obs.metrics import MetricsCollector
from ..ops import grpo_token_loss
from ..obs import nvtx
from ..optim import LRSchedule, ZeROOptimizer, build_optimizer
from ..pipeline import PipelineParallelContext, PipelineScheduler
from .icepop import IcePopConfig, IcePopFilter

logger = get_logger("train.engine")


@dataclass
class TrainConfig:
    model_path: str = ""
    tp_size: int = 1
    dp_size: int = 1
    pp_size: int = 1
    num_micro_batches: int = 1
    max_seq_len: int = 2048
    use_flash_attn: bool = False          # accepted for config compatibility; attention is always the
    attention_backend: str = "sdpa"       # native flash kernel on GPU
    use_gradient_checkpoint: bool = False
    cuda_graph_step: bool = False              # replay forward + backward of a micro-batch as one CUDA graph
    cuda_graph_reduce: Optional[bool] = None    # ... with the last micro-batch's gradient reduce-scatters captured in it
                                                # (None: yes for the in-kernel "p2p" ZeRO backend, no for NCCL)
    lora_rank: int = 16
    lora_alpha: float = 32.0
    lora_target_modules: List[str] = field(default_factory=lambda: [
        "q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj"])
    learning_rate: float = 1e-5
    weight_decay: float = 0.01
    max_grad_norm: float = 1.0
    use_amp: bool = True
    amp_dtype: str = "bf16"
    gradient_accumulation_steps: int = 4
    grpo_num_samples: int = 4
    grpo_beta: float = 0.1
    grpo_clip_eps: float = 0.2
    pad_token_id: int = 0
    zero_stage: int = 1
    enable_comm_overlap: bool = False
    min_prompt_len: int = 16
    lr_scheduler_type: str = "cosine"
    warmup_steps: int = 100
    min_lr_ratio: float = 0.1
    total_training_steps: int = 0
    icepop_enabled: bool = False
    icepop_divergence_threshold: float = 0.5
    icepop_max_mask_ratio: float = 0.5
    # ---- additions -------------------------------------------------------------------------------
    model_preset: Optional[str] = None          # random-init architecture from model.PRESETS
    model_config: Optional[ModelConfig] = None  # or an explicit architecture
    sequence_parallel: bool = False
    seed: int = 0
    adam_beta1: float = 0.9
    adam_beta2: float = 0.999
    adam_eps: float = 1e-8
    bucket_mb: float = 64.0
    fused_tp_comm: bool = False                 # TP+SP: all-gather / reduce-scatter inside the GEMM kernels
    zero_comm_backend: str = "auto"           # "p2p": reduce-scatter / all-gather inside the optimizer kernels over
                                                # peer memory / NVLS; "nccl": library collectives; "auto": p2p for plain
                                                # data parallelism with ZeRO-1 on 2..8 GPUs of a node, NCCL otherwise
    zero3_prefetch: bool = True                 # ZeRO-3: overlap the per-bucket parameter gathers with the forward
    build_ref_model: Optional[bool] = None      # default: grpo_beta > 0, as in the reference
    backend: Optional[str] = None               # nccl / gloo (default by device)
    heartbeat_interval_s: float = 0.0           # > 0: watch the other ranks over the rendezvous store and refuse to
    heartbeat_timeout_s: float = 10.0           # launch a step once one of them is gone (b200fw.dist.heartbeat)


@dataclass
class TrainMetrics:
    loss: float
    policy_loss: float
    kl_divergence: float
    grad_norm: float
    learning_rate: float
    step: int
    extras: Dict[str, float] = field(default_factory=dict)


class TrainEngine:
    def __init__(self, config: TrainConfig):
        self.config = config
        self.parallel_ctx: Optional[ParallelContext] = None
        self.model: Optional[ParallelTransformerModel] = None
        self.ref_model: Optional[ParallelTransformerModel] = None
        self.optimizer: Optional[ZeROOptimizer] = None
        self.lr_scheduler: Optional[LRSchedule] = None
        self.model_config: Optional[ModelConfig] = None
        self.step_count = 0
        self._accumulation_count = 0
        self.metrics_collector: Optional[MetricsCollector] = None
        self._old_log_probs_buffer: Optional[torch.Tensor] = None
        self.pp_context: Optional[PipelineParallelContext] = None
        self.pipeline_scheduler: Optional[PipelineScheduler] = None
        self.icepop: Optional[IcePopFilter] = None
        self.heartbeat = None                       # b200fw.dist.heartbeat.RankHeartbeat when enabled
        self._prev_lora_snapshot: Optional[Dict[str, torch.Tensor]] = None
        self.memory_profiler = MemoryProfiler()
        self.device = torch.device("cpu")
        self.dtype = torch.float32
        self._pinned: Dict[str, torch.Tensor] = {}
        self.last_icepop_info: Dict[str, float] = {}
        self.last_grpo_info: Dict[str, float] = {}
        self._graphs: Dict[tuple, dict] = {}          # (B, S, rows, first-of-window) -> captured micro-step
        self._graph_pool = None
        self._graph_seen: Dict[tuple, int] = {}
        self._graph_disabled = False
        self.last_h2d_bytes = 0                       # bytes the last sft_step_tensors call copied host -> device

    # =============================================================================================
    def initialize(self, parallel_context: Optional[ParallelContext] = None):
        cfg = self.config
        if parallel_context is not None:
            ctx = parallel_context
        elif int(os.environ.get("WORLD_SIZE", "1")) > 1 or cfg.tp_size * cfg.dp_size * cfg.pp_size > 1:
            ctx = ParallelContext.init_distributed(cfg.tp_size, cfg.dp_size, cfg.pp_size, cfg.backend)
        else:
            ctx = ParallelContext.init_single_process()
        self.parallel_ctx = ctx
        self.device = ctx.device
        if self.device.type == "cuda":
            from .. import _native
            _native.set_device(self.device.index or 0)
        if cfg.pp_size > 1:
            if cfg.zero_stage > 1:
                raise ValueError("pipeline parallelism supports zero_stage <= 1")
            if cfg.num_micro_batches < cfg.pp_size:
                raise ValueError("num_micro_batches must be >= pp_size")
        amp = cfg.amp_dtype if cfg.use_amp else "fp32"
        if amp == "fp16":
            logger.warning("precision fp16 runs as bf16: the kernels are bf16-only (and bf16 needs no loss scaling)")
        self.dtype = {"bf16": torch.bfloat16, "fp16": torch.bfloat16, "fp32": torch.float32}[amp]
        if self.device.type == "cpu":
            self.dtype = torch.float32 if amp == "fp32" or not cfg.use_amp else self.dtype
        # ---- architecture ----------------------------------------------------------------------
        if cfg.model_config is not None:
            mc = cfg.model_config
        elif cfg.model_preset is not None:
            mc = copy.deepcopy(PRESETS[cfg.model_preset])
        else:
            mc = read_hf_config(cfg.model_path)
        self.model_config = mc
        if cfg.max_seq_len > mc.max_position_embeddings:
            # sequences are truncated to max_seq_len when batches are built: truncate to what the model can address
            logger.warning("max_seq_len=%d exceeds the model's max_position_embeddings=%d: using %d", cfg.max_seq_len,
                           mc.max_position_embeddings, mc.max_position_embeddings)
            cfg.max_seq_len = mc.max_position_embeddings
        layer_range, first, last = None, True, True
        if cfg.pp_size > 1:
            if mc.num_layers < cfg.pp_size:
                raise ValueError(f"{mc.num_layers} layers cannot fill {cfg.pp_size} pipeline stages")
            self.pp_context = PipelineParallelContext(mc.num_layers, ctx)
            layer_range = (self.pp_context.layer_start, self.pp_context.layer_end)
            first, last = self.pp_context.is_first_stage, self.pp_context.is_last_stage
            if mc.tie_word_embeddings:
                mc = copy.deepcopy(mc)
                mc.tie_word_embeddings = False  # the two ends live on different stages
                self.model_config = mc
        self.model = ParallelTransformerModel(
            mc, ctx, layer_range, first, last, sequence_parallel=cfg.sequence_parallel,
            gradient_checkpointing=cfg.use_gradient_checkpoint, dtype=self.dtype, device=self.device)
        self.model.init_weights(cfg.seed)
        # `enable_comm_overlap` is the reference's switch for overlapping tensor-parallel communication with
        # compute (its async MLP all-reduce: src/distributed/tensor_parallel.py:718-720); here the overlap is
        # the fused all-gather -> GEMM / GEMM -> reduce-scatter kernels, which need the sequence-parallel layout
        if ((cfg.fused_tp_comm or cfg.enable_comm_overlap) and cfg.sequence_parallel and cfg.tp_size > 1
                and self.device.type == "cuda"):
            self.model.set_fused_comm(True)
        if cfg.model_path and os.path.isdir(cfg.model_path):
            loaded, missing = load_from_hf_checkpoint(self.model, cfg.model_path)
            logger.info("loaded %d tensors from %s (%d missing)", loaded, cfg.model_path, missing)
        # ---- frozen reference policy ---------------------------------------------------------------
        want_ref = cfg.build_ref_model if cfg.build_ref_model is not None else cfg.grpo_beta > 0
        if want_ref and cfg.lora_rank <= 0 and cfg.pp_size == 1:
            self.ref_model = self.model.clone(requires_grad=False)
            self.ref_model.eval()
        self._ref_is_base = bool(want_ref and cfg.lora_rank > 0)  # LoRA: reference = adapters off
        # ---- LoRA -------------------------------------------------------------------------------
        if cfg.lora_rank > 0:
            names = apply_lora(self.model, cfg.lora_rank, cfg.lora_alpha, cfg.lora_target_modules)
            logger.info("LoRA r=%d on %d projections", cfg.lora_rank, len(names))
        # ---- optimizer + schedule -------------------------------------------------------------------
        trainable = [p for p in self.model.parameters() if p.requires_grad]
        self.optimizer = build_optimizer(
            trainable, cfg.zero_stage if (cfg.dp_size > 1 or cfg.tp_size > 1 or cfg.zero_stage == 0) else 1,
            lr=cfg.learning_rate, betas=(cfg.adam_beta1, cfg.adam_beta2), eps=cfg.adam_eps,
            weight_decay=cfg.weight_decay, ctx=ctx, bucket_mb=cfg.bucket_mb, max_grad_norm=cfg.max_grad_norm,
            overlap=True, comm_backend=cfg.zero_comm_backend)
        if cfg.zero3_prefetch:
            self.optimizer.attach_prefetch_hooks(self.model)  # ZeRO-3 on a GPU: parameter gathers overlap the forward
        self.lr_scheduler = LRSchedule(cfg.learning_rate, cfg.lr_scheduler_type, cfg.warmup_steps,
                                       cfg.total_training_steps, cfg.min_lr_ratio)
        self.optimizer.param_groups[0]["lr"] = self.lr_scheduler.lr_at(0)
        ctx.on_destroy(self.release_graphs)
        if cfg.heartbeat_interval_s > 0:
            from ..dist.heartbeat import RankHeartbeat
            self.heartbeat = RankHeartbeat.from_default_group(cfg.heartbeat_interval_s, cfg.heartbeat_timeout_s)
            if self.heartbeat is not None:
                self.heartbeat.start()
                ctx.on_destroy(self.heartbeat.announce_leave)      # leaving on purpose is not a failure
        if cfg.pp_size > 1:
            self.pipeline_scheduler = PipelineScheduler(self.model, self.pp_context, cfg.num_micro_batches)
        if cfg.icepop_enabled:
            self.icepop = IcePopFilter(IcePopConfig(True, cfg.icepop_divergence_threshold, cfg.icepop_max_mask_ratio))
        self.memory_profiler.snapshot("after_init")
        return self

    # ---- batching ------------------------------------------------------------------------------
    def _truncate_prompt_response(self, prompt: List[int], response: List[int]) -> Tuple[List[int], List[int]]:
        """Fit ``prompt + response`` into ``max_seq_len``: keep the response if possible (it is the
        training target) and trim the prompt's tail; if the response alone is too long, cut it and keep
        ``min_prompt_len`` prompt tokens."""
        L = self.config.max_seq_len
        keep = min(self.config.min_prompt_len, len(prompt))
        if len(prompt) + len(response) <= L:
            return prompt, response
        if len(response) >= L - keep:
            return prompt[:keep], response[:L - keep]
        return prompt[:L - len(response)], response

    def _pinned_buf(self, name: str, numel: int) -> torch.Tensor:
        """A reusable pinned int64 staging buffer (page-locking memory per call costs more than the copy)."""
        buf = self._pinned.get(name)
        if buf is None or buf.numel() < numel:
            buf = torch.empty(max(numel, 1), dtype=torch.long, pin_memory=True)
            self._pinned[name] = buf
        return buf[:numel]

    def _check_peers(self):
        """Before anything of a step is launched: if the heartbeat watcher has found a rank gone, raise
        ``PeerLostError`` here instead of entering collectives (or peer-memory kernels) that rank will never join."""
        if self.heartbeat is not None:
            self.heartbeat.check()

    def _check_host_batch(self, input_ids: Optional[torch.Tensor], labels: Optional[torch.Tensor] = None):
        """Refuse token ids and labels outside the vocabulary, and rows longer than the position table, while the
        batch is still in host memory: the embedding, rotary and loss kernels index their tables with these values
        unchecked, so a bad id would read outside the table on the device.  Device tensors are not inspected (that
        would cost a synchronisation); their producer is responsible for them."""
        mc = self.model_config
        if mc is None:
            return
        V = mc.vocab_size
        if input_ids is not None and input_ids.device.type == "cpu" and input_ids.numel():
            lo, hi = int(input_ids.min()), int(input_ids.max())
            if lo < 0 or hi >= V:
                raise ValueError(f"token id {lo if lo < 0 else hi} is outside the vocabulary [0, {V})")
            if input_ids.shape[-1] > mc.max_position_embeddings:
                raise ValueError(f"sequence length {input_ids.shape[-1]} exceeds max_position_embeddings="
                                 f"{mc.max_position_embeddings}")
        if labels is not None and labels.device.type == "cpu" and labels.numel():
            hi = int(labels.max())
            bad_neg = int(((labels < 0) & (labels != -100)).sum())
            if hi >= V or bad_neg:
                raise ValueError(f"labels must be token ids in [0, {V}) or -100 (largest {hi}, "
                                 f"{bad_neg} negative values other than -100)")

    def _to_device(self, name: str, rows: List[List[int]], fill: int, on_host: bool = False) -> torch.Tensor:
        """Pad ``rows`` to a rectangle in a reusable pinned host buffer and copy it to the device
        (``on_host``: hand back the pinned view itself; the caller copies)."""
        n, m = len(rows), max(len(r) for r in rows)
        if self.device.type != "cuda":
            t = torch.full((n, m), fill, dtype=torch.long)
            for i, r in enumerate(rows):
                t[i, :len(r)] = torch.tensor(r, dtype=torch.long)
            self._check_host_batch(t if name == "ids" else None, t if name == "labels" else None)
            return t
        view = self._pinned_buf(name, n * m).view(n, m)
        if all(len(r) == m for r in rows):
            view.copy_(torch.tensor(rows, dtype=torch.long))          # one conversion for a rectangular batch
        else:
            view.fill_(fill)
            for i, r in enumerate(rows):
                view[i, :len(r)] = torch.tensor(r, dtype=torch.long)
        self._check_host_batch(view if name == "ids" else None, view if name == "labels" else None)
        return view if on_host else view.to(self.device, non_blocking=True)

    def _build_batch(self, prompts: List[List[int]], responses: List[List[int]], on_host: bool = False):
        ids, labels = [], []
        for p, r in zip(prompts, responses):
            p, r = self._truncate_prompt_response(list(p), list(r))
            ids.append(p + r)
            labels.append([-100] * len(p) + r)
        return (self._to_device("ids", ids, self.config.pad_token_id, on_host),
                self._to_device("labels", labels, -100, on_host))

    # ---- optimizer step --------------------------------------------------------------------------
    def _maybe_step(self, skip: bool = False):
        """After ``gradient_accumulation_steps`` backwards: clip (global norm), AdamW, schedule."""
        cfg = self.config
        if self._accumulation_count < cfg.gradient_accumulation_steps or skip:
            return None
        opt = self.optimizer
        opt.param_groups[0]["lr"] = self.lr_scheduler.get_last_lr()[0]
        with nvtx.range("train/reduce_and_clip"):
            gn = opt.clip_grad_norm(cfg.max_grad_norm)
        with nvtx.range("train/adamw_and_publish"):
            opt.step()           # the kernel itself skips the update when the norm is not finite
        opt.zero_grad()
        self._accumulation_count = 0
        return gn

    def _check_device_status(self):
        """Read the kernels' status word once per optimizer step, at a host sync that exists anyway.  A bounded
        device wait that ran out (a peer's gradient flag, a GEMM / attention pipeline barrier) leaves a code
        there and returns; without this check training would go on over whatever the abandoned kernel left."""
        if self.device.type != "cuda":
            return
        from .. import _native as nv
        st = nv.read_status()
        if st != 0:
            flags = getattr(self.optimizer, "flags", None)
            if flags is not None:
                flags.reset_ok()        # the failed step's update was skipped on the device; later steps may proceed
            raise nv.NativeError(f"device status {st} after optimizer step {self.step_count}: a bounded wait in a "
                                 "kernel ran out (301: a peer's flag never arrived; 1xx/2xx: a pipeline barrier); "
                                 "the update of this step is not trustworthy")

    def _clip_grad_norm(self) -> float:
        """Global L2 norm of the gradients over DP x TP x PP, with the clip to ``max_grad_norm`` armed for the next
        ``optimizer.step()``; ``-1.0`` when the norm is not finite (the step then leaves the weights untouched).
        The reference's unit of the same name (src/engines/train_engine.py:1451-1530) scales ``p.grad`` in place;
        here the scale is applied inside the fused AdamW kernel, so the gradients themselves stay as they are.

        An object without a bucketed optimizer (a bare model whose gradients sit in ``p.grad``: the form the
        reference's ``tests/test_grad_norm_3d.py`` drives with a stub engine) gets the plain form: the sum of squares
        of the local gradients is all-reduced over every parallel group that has more than one rank, gradients of
        parameters marked ``_tp_replicated`` are first summed over TP, and ``p.grad`` is scaled in place when the
        norm exceeds ``max_grad_norm``."""
        opt = getattr(self, "optimizer", None)
        if opt is not None and hasattr(opt, "clip_grad_norm"):
            return float(opt.clip_grad_norm(self.config.max_grad_norm))
        params = [p for p in self.model.parameters() if p.requires_grad and p.grad is not None]
        if not params:
            return 0.0
        ctx = getattr(self, "parallel_ctx", None)
        if ctx is not None and ctx.tp_size > 1 and ctx.tp_group is not None:
            for p in params:
                if getattr(p, "_tp_replicated", False):
                    dist.all_reduce(p.grad, group=ctx.tp_group)
        sq = torch.stack([p.grad.detach().double().pow(2).sum() for p in params]).sum()
        if ctx is not None and ctx.world_size > 1:
            for size, group in ((ctx.dp_size, ctx.dp_group), (ctx.tp_size, ctx.tp_group), (ctx.pp_size, ctx.pp_group)):
                if size > 1 and group is not None:
                    dist.all_reduce(sq, group=group)
        if not bool(torch.isfinite(sq)):       # after the reductions: a NaN on one rank reaches all, nobody leaves early
            return -1.0
        norm = float(sq.sqrt())
        scale = float(self.config.max_grad_norm) / (norm + 1e-6)
        if scale < 1.0:
            torch._foreach_mul_([p.grad for p in params], scale)
        mc = getattr(self, "metrics_collector", None)
        if mc is not None:
            mc.record("grad_norm", norm)
        return norm

    def _finish_step(self, gn: Optional[torch.Tensor]) -> float:
        """Host side of the NaN/Inf guard: a non-finite norm (reported as -1) means the device skipped
        the update, so neither the step counter nor the schedule advance."""
        if gn is None:
            return 0.0
        g = float(gn)
        self._check_device_status()
        if g < 0:
            logger.warning("non-finite gradient norm: optimizer step skipped")
            self.optimizer.step_count -= 1
            return g
        self.lr_scheduler.step()
        self.step_count += 1
        if self.metrics_collector is not None:
            self.metrics_collector.record("grad_norm", g)
        return g

    # =============================================================================================
    def sft_step(self, prompts_tokens: List[List[int]], response_tokens: List[List[int]]) -> TrainMetrics:
        """Teacher-forced SFT step; prompt positions are not supervised."""
        # on a GPU the batch stays in pinned host memory until sft_step_tensors ships it together with the
        # supervised-row indices (known on the host, so the LM head needs no device -> host count)
        ids, labels = self._build_batch(prompts_tokens, response_tokens, on_host=self.device.type == "cuda")
        return self.sft_step_tensors(ids, labels, _checked=True)        # _build_batch has looked at the values

    def sft_step_tensors(self, input_ids: torch.Tensor, labels: torch.Tensor, sync: bool = True, _checked: bool = False):
        """SFT step on ready ``[B,S]`` tensors (host tensors are copied to the device asynchronously).
        ``sync=False`` returns ``(loss_tensor, grad_norm_tensor_or_None)`` without a host sync."""
        valid_idx = None
        self._check_peers()
        if not _checked:
            self._check_host_batch(input_ids, labels)
        if input_ids.device != self.device:
            if labels.device.type == "cpu" and self.device.type == "cuda":
                # the supervised rows (label of the next token is not -100) are known on the host before the
                # copy: ship their indices along, so the LM head never needs a device -> host count
                nxt = torch.full_like(labels, -100)
                nxt[:, :-1] = labels[:, 1:]
                idx = torch.nonzero(nxt.reshape(-1) != -100).squeeze(-1)
                if idx.numel() < nxt.numel():
                    if sync:    # this call ends with a host sync, so the staging buffer is free again next call
                        stage = self._pinned_buf("valid_idx", idx.numel())
                        stage.copy_(idx)
                    else:
                        stage = idx.pin_memory()
                    valid_idx = stage.to(self.device, non_blocking=True)
                self.last_h2d_bytes = 8 * (input_ids.numel() + labels.numel() + (idx.numel() if valid_idx is not None else 0))
            input_ids = input_ids.to(self.device, non_blocking=True)
            labels = labels.to(self.device, non_blocking=True)
        if self.pp_context is not None and self.pp_context.pp_size > 1:
            loss, gn = self._pp_batch_step(input_ids, labels)
        else:
            loss, gn = self._single_batch_step(input_ids, labels, valid_idx)
        if not sync:
            if gn is not None:   # optimistic bookkeeping; resolve_step(gn) applies the NaN guard later
                self.lr_scheduler.step()
                self.step_count += 1
            return loss, gn
        lr = self.lr_scheduler.get_last_lr()[0]
        g = self._finish_step(gn)
        lv = float(loss)
        if self.metrics_collector is not None:
            self.metrics_collector.record("learning_rate", lr)
            self.metrics_collector.record("loss", lv)
        return TrainMetrics(lv, lv, 0.0, g, lr, self.step_count)

    def resolve_step(self, gn: Optional[torch.Tensor]) -> float:
        """Settle one ``sft_step_tensors(..., sync=False)`` optimizer step after the fact (this synchronises):
        reads the norm, checks the device status word, and when the norm was not finite (the device skipped
        AdamW) takes back the optimistic bookkeeping: the optimizer's bias-correction step, the schedule and
        the step counter.  Call it in step order, before the learning rate of a later step matters.  Returns the
        gradient norm (``-1`` for a skipped step, ``0`` when ``gn`` is ``None``: no optimizer step happened)."""
        if gn is None:
            return 0.0
        g = float(gn)
        self._check_device_status()
        if g < 0:
            logger.warning("non-finite gradient norm: optimizer step skipped")
            self.optimizer.step_count = max(0, self.optimizer.step_count - 1)
            self.lr_scheduler.step_count = max(0, self.lr_scheduler.step_count - 1)
            self.step_count = max(0, self.step_count - 1)
        elif self.metrics_collector is not None:
            self.metrics_collector.record("grad_norm", g)
        return g

    def close_accumulation_window(self) -> TrainMetrics:
        """Run the optimizer step now, over however many micro-batches have been accumulated (C3PO++ packs a
        batch into a variable number of chunks; the last chunk closes the window).  No-op when nothing is
        pending."""
        lr = self.lr_scheduler.get_last_lr()[0]
        if self._accumulation_count == 0:
            return TrainMetrics(0.0, 0.0, 0.0, 0.0, lr, self.step_count)
        self._accumulation_count = max(self._accumulation_count, self.config.gradient_accumulation_steps)
        g = self._finish_step(self._maybe_step())
        return TrainMetrics(0.0, 0.0, 0.0, g, lr, self.step_count)

    def _single_batch_step(self, input_ids, labels, valid_idx=None):
        cfg, opt = self.config, self.optimizer
        opt.pre_forward(lazy=True)
        if self._graph_eligible():
            with nvtx.range("train/micro_step/graph"):
                loss = self._graphed_micro_step(input_ids, labels, valid_idx)
            if loss is not None:
                opt.post_backward()
                self._accumulation_count += 1
                return loss, self._maybe_step()
        opt.begin_backward(sync=self._accumulation_count + 1 >= cfg.gradient_accumulation_steps)
        with nvtx.range("train/micro_step/forward"):
            loss = self.model.loss(input_ids, labels, loss_scale=1.0 / cfg.gradient_accumulation_steps,
                                   valid_idx=valid_idx)
        with nvtx.range("train/micro_step/backward"):
            loss.backward()
        opt.post_backward()
        self._accumulation_count += 1
        return loss.detach(), self._maybe_step()

    @property
    def trainable_params_count(self) -> int:
        """Trainable parameters on this rank (src/engines/train_engine.py:1756-1768)."""
        return 0 if self.model is None else sum(p.numel() for p in self.model.parameters() if p.requires_grad)

    @property
    def total_params_count(self) -> int:
        return 0 if self.model is None else sum(p.numel() for p in self.model.parameters())

    # ---- CUDA-graph micro-step ----------------------------------------------------------------------
    def release_graphs(self):
        """Drop every captured micro-step graph (and the memory pool they share).  Graphs that contain
        reduce-scatters hold references on the NCCL communicator, which cannot be destroyed before them;
        the parallel context calls this ahead of its own teardown."""
        if self._graphs:
            if self.device.type == "cuda":
                torch.cuda.synchronize()
            self._graphs.clear()
            self._graph_pool = None
            if self.optimizer is not None:
                self.optimizer._reduced_shards.clear()      # may point into the released pool
            import gc
            gc.collect()
            if self.device.type == "cuda":
                torch.cuda.synchronize()

    def _graph_eligible(self) -> bool:
        cfg, opt = self.config, self.optimizer
        return (cfg.cuda_graph_step and not self._graph_disabled and self.device.type == "cuda"
                and cfg.tp_size == 1 and cfg.pp_size == 1 and not cfg.use_gradient_checkpoint
                and getattr(opt, "stage", 0) <= 1 and getattr(opt, "use_main_grad", False))

    def _graphed_micro_step(self, input_ids, labels, valid_idx):
        """Forward + loss + backward of one micro-batch as a replayed CUDA graph.

        About 800 kernels are launched per micro-batch; launched one by one the GPU idles ~10 % of the step
        between them.  The graph is keyed by the batch shape, the (padded) number of supervised rows and
        whether this is the first micro-batch of the accumulation window (the weight-gradient GEMMs then
        overwrite instead of accumulating).  Gradients land in the optimizer's persistent bucket buffers, so
        reduction, clipping and AdamW stay outside the graph.  The first two micro-batches of a key run
        eagerly (lazy initialisation, allocator warm-up), the third is captured.  Returns ``None`` when
        the step has to run eagerly."""
        from .. import _native as nv
        cfg, opt = self.config, self.optimizer
        B, S = input_ids.shape
        shifted = torch.full_like(labels, -100)
        shifted[:, :-1] = labels[:, 1:]
        shifted = shifted.reshape(-1)
        if valid_idx is None:
            valid_idx = torch.nonzero(shifted != -100).squeeze(-1)     # device labels: one host sync
        n = int(valid_idx.numel())
        if n == 0:
            return None
        rows = -(-n // 512) * 512                                       # bucket the row count
        first = self._accumulation_count == 0
        # last micro-batch of the window on several data-parallel ranks: the bucket reduce-scatters are captured
        # too, on the optimizer's side stream, so they overlap the rest of the backward pass inside the graph
        want = cfg.cuda_graph_reduce if cfg.cuda_graph_reduce is not None else bool(getattr(opt, "p2p", False))
        reduce_in_graph = (want and opt.world > 1 and opt.stage == 1
                           and self._accumulation_count + 1 >= cfg.gradient_accumulation_steps)
        key = (B, S, rows, first, reduce_in_graph)
        seen = self._graph_seen.get(key, 0)
        self._graph_seen[key] = seen + 1
        if seen < 2:
            return None
        g = self._graphs.get(key)
        if g is None:
            g = {"ids": torch.zeros_like(input_ids), "idx": torch.zeros(rows, dtype=torch.long, device=self.device),
                 "lab": torch.full((rows,), -100, dtype=torch.long, device=self.device)}
        g["ids"].copy_(input_ids)
        g["idx"].zero_()
        g["idx"][:n].copy_(valid_idx)
        g["lab"].fill_(-100)                                            # padding rows carry no label
        g["lab"][:n].copy_(shifted.index_select(0, valid_idx))
        if "graph" not in g:
            # the gradient hooks launch reductions inside the capture only when they are meant to be part of it
            opt.begin_backward(sync=reduce_in_graph)
            before = nv.launch_count
            try:
                torch.cuda.synchronize()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, pool=self._graph_pool):
                    loss = self.model.loss(g["ids"], None, loss_scale=1.0 / cfg.gradient_accumulation_steps,
                                           valid_idx=g["idx"], valid_labels=g["lab"])
                    loss.backward()
                    g["loss"] = loss.detach()
                    if reduce_in_graph:
                        g["reduced"] = opt.finish_captured_reduces()
            except Exception as e:  # noqa: BLE001 - fall back to eager for good
                logger.warning("CUDA-graph capture of the training micro-step failed (%s): running eagerly", e)
                self._graph_disabled = True
                opt.abandon_captured_reduces()
                torch.cuda.synchronize()
                return None
            if self._graph_pool is None:
                self._graph_pool = graph.pool()
            g["graph"], g["launches"] = graph, nv.launch_count - before
            self._graphs[key] = g
        else:
            nv.count_launch(g["launches"])
        g["graph"].replay()
        # the replay bypasses the Python-side gradient hooks: record that every bucket now holds gradients
        # (a later eager or newly captured micro-step of this window must accumulate, not overwrite)
        for b in opt.buckets:
            for p in b.params:
                p.grad_filled = True
        if g.get("reduced") is not None:
            opt.adopt_reduced(g["reduced"])
        return g["loss"].clone()

    def _pp_batch_step(self, input_ids, labels):
        cfg, opt = self.config, self.optimizer
        opt.begin_backward(sync=True, backward_passes=cfg.num_micro_batches)
        loss = self.pipeline_scheduler.run_1f1b_schedule(input_ids, labels)
        opt.post_backward()
        self._accumulation_count = cfg.gradient_accumulation_steps
        gn = self._maybe_step()
        return self.pipeline_scheduler.broadcast_loss(loss), gn

    @torch.no_grad()
    def eval_sft_loss(self, prompts_tokens: List[List[int]], response_tokens: List[List[int]]) -> float:
        ids, labels = self._build_batch(prompts_tokens, response_tokens)
        with self.optimizer.eval_mode():
            was = self.model.training
            self.model.eval()
            try:
                return float(self.model.loss(ids, labels))
            finally:
                self.model.train(was)

    # =============================================================================================
    @staticmethod
    def group_advantages(rewards: List[float]) -> List[float]:
        """Group-normalised advantages; all-equal rewards carry no signal and give zeros."""
        t = torch.tensor(rewards, dtype=torch.float32)
        std = t.std(unbiased=False)
        if std < 1e-8:
            return [0.0] * len(rewards)
        return ((t - t.mean()) / (std + 1e-8)).tolist()

    def _lora_enabled(self, on: bool):
        for m in self.model.modules():
            if isinstance(m, LinearWithLoRA):
                m.merged = not on   # `merged=True` bypasses the adapters in forward

    @torch.no_grad()
    def _ref_token_logprobs(self, ids, labels) -> Optional[torch.Tensor]:
        if self.ref_model is not None:
            return self.ref_model.token_logprobs(ids, labels=labels)
        if self._ref_is_base:
            self._lora_enabled(False)
            try:
                return self.model.token_logprobs(ids, labels=labels)
            finally:
                self._lora_enabled(True)
        return None

    def grpo_step(self, prompts_tokens: List[List[int]], responses_group: List[List[List[int]]],
                  rewards_group: List[List[float]], infer_log_probs: Optional[torch.Tensor] = None,
                  skip_optimizer_step: bool = False, reset_behavior_baseline: bool = True,
                  precomputed_advantages: Optional[List[List[float]]] = None,
                  close_window: bool = False) -> TrainMetrics:
        """One GRPO step over ``batch x K`` sequences: group-relative advantages, clipped token-level
        surrogate against the behaviour log-probs, KL to the frozen reference, optional IcePop.
        ``close_window`` makes this backward the last of the accumulation window whatever the count says
        (C3PO++ packs a batch into a variable number of chunks and closes the window on the last one)."""
        assert self.pp_context is None or self.pp_context.pp_size == 1, "GRPO needs pp_size == 1"
        self._check_peers()
        cfg, opt = self.config, self.optimizer
        if reset_behavior_baseline:
            self._old_log_probs_buffer = None
        P, R, A = [], [], []
        for i, prompt in enumerate(prompts_tokens):
            adv = precomputed_advantages[i] if precomputed_advantages is not None \
                else self.group_advantages(rewards_group[i])
            for k, resp in enumerate(responses_group[i]):
                P.append(prompt)
                R.append(resp)
                A.append(adv[k])
        ids, labels = self._build_batch(P, R)
        adv_t = torch.tensor(A, dtype=torch.float32).to(self.device, non_blocking=True)
        mask = (labels[:, 1:] != -100).float()
        opt.pre_forward(lazy=True)
        if close_window:
            self._accumulation_count = max(self._accumulation_count, cfg.gradient_accumulation_steps - 1)
        opt.begin_backward(sync=self._accumulation_count + 1 >= cfg.gradient_accumulation_steps)
        lp = self.model.token_logprobs(ids, labels=labels)
        self.last_icepop_info = {}
        if self.icepop is not None and self.icepop.config.enabled:
            seq_lp = (lp.detach() * mask).sum(-1) / (mask.sum(-1) + 1e-8)
            if infer_log_probs is None:
                infer_log_probs = self._inference_log_probs(ids, labels, mask)
            adv_t, self.last_icepop_info = self.icepop.filter_divergent_responses(seq_lp, infer_log_probs, adv_t)
        ref_lp = self._ref_token_logprobs(ids, labels) if cfg.grpo_beta > 0 else None
        old_lp = lp.detach() if self._old_log_probs_buffer is None or \
            self._old_log_probs_buffer.shape != lp.shape else self._old_log_probs_buffer
        loss, info = grpo_token_loss(lp, old_lp, ref_lp, mask, adv_t, cfg.grpo_clip_eps, cfg.grpo_beta,
                                     loss_scale=1.0 / cfg.gradient_accumulation_steps)
        self._old_log_probs_buffer = lp.detach().clone()
        loss.backward()
        opt.post_backward()
        self._accumulation_count += 1
        gn = self._maybe_step(skip=skip_optimizer_step)
        lr = self.lr_scheduler.get_last_lr()[0]
        g = self._finish_step(gn)
        self.last_grpo_info = {k: float(v) for k, v in info.items()}
        if self.metrics_collector is not None:
            self.metrics_collector.record("learning_rate", lr)
        return TrainMetrics(float(loss.detach()), self.last_grpo_info["policy_loss"], self.last_grpo_info["kl_divergence"],
                            g, lr, self.step_count, extras={**self.last_grpo_info, **self.last_icepop_info})

    @torch.no_grad()
    def _inference_log_probs(self, ids, labels, mask) -> torch.Tensor:
        """Sequence log-probs from an inference-mode forward (the IcePop fallback when the rollout
        engine did not report its own)."""
        was = self.model.training
        self.model.eval()
        try:
            lp = self.model.token_logprobs(ids, labels=labels)
        finally:
            self.model.train(was)
        return (lp * mask).sum(-1) / (mask.sum(-1) + 1e-8)

    @torch.no_grad()
    def compute_sequence_log_probs(self, prompts_tokens, response_tokens) -> torch.Tensor:
        ids, labels = self._build_batch(prompts_tokens, response_tokens)
        mask = (labels[:, 1:] != -100).float()
        with self.optimizer.eval_mode():
            return self._inference_log_probs(ids, labels, mask)

    # =============================================================================================
    @staticmethod
    def sample_next_token(logits: torch.Tensor, temperature: float, top_p: float,
                          generator: Optional[torch.Generator] = None) -> torch.Tensor:
        """Temperature + nucleus sampling on ``[B,V]`` logits (greedy when ``temperature <= 0``)."""
        if temperature <= 0:
            return logits.argmax(-1)
        probs = torch.softmax(logits.float() / temperature, dim=-1)
        if top_p < 1.0:
            sp, si = probs.sort(dim=-1, descending=True)
            keep = (sp.cumsum(-1) - sp) < top_p      # keep the token that crosses the threshold
            keep[..., 0] = True                      # top_p <= 0: the most likely token alone
            sp = sp * keep
            probs = torch.zeros_like(probs).scatter_(-1, si, sp)
            probs = probs / probs.sum(-1, keepdim=True)
        return torch.multinomial(probs, 1, generator=generator).squeeze(-1)

    @torch.no_grad()
    def generate(self, prompt_tokens: List[int], max_new_tokens: int = 128, temperature: float = 0.7,
                 top_p: float = 0.95, eos_token_id: Optional[int] = None) -> List[int]:
        """Reference-compatible local generation: full re-forward per token, no KV cache
        (src/engines/train_engine.py:907-1008).  Kept for previews and tests; rollouts use
        :class:`b200fw.infer.InferenceEngine`.  Under TP, rank 0 of the TP group samples and broadcasts."""
        import torch.distributed as dist
        ctx = self.parallel_ctx
        seq = [int(t) for t in prompt_tokens]
        if not seq:
            raise ValueError("generate(): empty prompt")
        V = self.model_config.vocab_size
        if min(seq) < 0 or max(seq) >= V:
            raise ValueError(f"generate(): token id {min(seq) if min(seq) < 0 else max(seq)} is outside the vocabulary [0, {V})")
        out: List[int] = []
        with self.optimizer.eval_mode():
            was = self.model.training
            self.model.eval()
            try:
                for _ in range(max_new_tokens):
                    ids = torch.tensor([seq[-self.config.max_seq_len:]], dtype=torch.long, device=self.device)
                    logits = self.model(ids)[:, -1, :]
                    tok = self.sample_next_token(logits, temperature, top_p)
                    if ctx.tp_size > 1:
                        dist.broadcast(tok, src=ctx.tp_ranks[0], group=ctx.tp_group)
                    t = int(tok)
                    out.append(t)
                    seq.append(t)
                    if eos_token_id is not None and t == eos_token_id:
                        break
            finally:
                self.model.train(was)
        return out

    # =============================================================================================
    @torch.no_grad()
    def export_weights(self, device: Optional[str] = None) -> Dict[str, torch.Tensor]:
        """HF-named full weights with LoRA merged (TP shards gathered); stage-3 gathers first."""
        from ..model.hf_io import hf_named_tensors
        with self.optimizer.eval_mode():
            # merged tensors are built out of place: the frozen base weights (also the KL reference under LoRA)
            # must come out of an export bit-identical
            out = {k: (v.to(device) if device else v).clone()
                   for k, v in hf_named_tensors(self.model, merge_lora=True)}
        return out

    @torch.no_grad()
    def export_lora_delta(self, device: Optional[str] = None) -> Dict[str, torch.Tensor]:
        """Current LoRA tensors minus the previous export's snapshot (the first call returns the full
        state), on ``device`` when given.  Feeds the SwiftSync delta path."""
        cur = {k: (v.clone() if device is None else v.to(device, copy=True)) for k, v in get_lora_state_dict(self.model).items()}
        if self._prev_lora_snapshot is None:
            delta = {k: v.clone() for k, v in cur.items()}
        else:
            delta = {k: v - self._prev_lora_snapshot[k] for k, v in cur.items()}
        self._prev_lora_snapshot = cur
        return delta

    # ---- checkpoints --------------------------------------------------------------------------------
    @staticmethod
    def _atomic_save(obj, dest: str, as_json: bool = False):
        """Write beside the destination and rename over it: a reader (or a restart after a crash in the middle of a
        save) sees the previous file or the new one, never a torn one."""
        tmp = f"{dest}.tmp{os.getpid()}"
        if as_json:
            with open(tmp, "w") as f:
                json.dump(obj, f)
        else:
            torch.save(obj, tmp)
        os.replace(tmp, dest)

    def save_checkpoint(self, path: str, save_base_weights: Optional[bool] = None) -> None:
        """``lora_weights.pt`` + ``optimizer_state_rank{r}.pt`` (every rank saves its own shard; rank 0
        also writes the reference-compatible ``optimizer_state.pt``) + HF-format base weights for full fine-tuning +
        ``trainer_state.json`` (step counters, LR schedule, RNG).  Every file is written atomically, and the state
        file last, after all ranks have finished theirs: its step count names the step every other file belongs to."""
        ctx = self.parallel_ctx
        os.makedirs(path, exist_ok=True)
        rank = ctx.global_rank
        lora = get_lora_state_dict(self.model)
        if lora and ctx.dp_rank == 0:
            name = "lora_weights.pt" if ctx.tp_size == 1 else f"lora_weights_tp{ctx.tp_rank}.pt"
            self._atomic_save({k: v.cpu() for k, v in lora.items()}, os.path.join(path, name))
        sd = self.optimizer.state_dict()
        sd["trainer_step"] = self.step_count
        self._atomic_save(sd, os.path.join(path, f"optimizer_state_rank{rank}.pt"))
        if rank == 0:
            self._atomic_save(sd, os.path.join(path, "optimizer_state.pt"))
        full = save_base_weights if save_base_weights is not None else (self.config.lora_rank <= 0)
        if full:
            with self.optimizer.eval_mode():
                shard = "model.safetensors" if ctx.pp_size == 1 else f"model-stage{ctx.pp_rank}.safetensors"
                save_hf_checkpoint(self.model, path, write=(ctx.dp_rank == 0 and ctx.tp_rank == 0), shard_name=shard)
        ctx.barrier()
        if rank == 0:
            self._atomic_save({"step_count": self.step_count, "accumulation_count": self._accumulation_count,
                               "lr_scheduler": self.lr_scheduler.state_dict(), "world_size": ctx.world_size,
                               "torch_rng_seed": int(torch.initial_seed())},
                              os.path.join(path, "trainer_state.json"), as_json=True)
        ctx.barrier()

    def _read_checkpoint(self, path: str) -> Dict[str, object]:
        """The local half of a restore: read this rank's files and check them against this run, touching neither the
        model nor the optimizer and calling no collective."""
        ctx = self.parallel_ctx
        out: Dict[str, object] = {"weights": False, "lora": None, "opt": None, "state": None}
        out["weights"] = self.config.lora_rank <= 0 and any(f.endswith(".safetensors") for f in os.listdir(path))
        lname = "lora_weights.pt" if ctx.tp_size == 1 else f"lora_weights_tp{ctx.tp_rank}.pt"
        lpath = os.path.join(path, lname)
        if os.path.exists(lpath):
            out["lora"] = torch.load(lpath, map_location="cpu", weights_only=True)
        spath = os.path.join(path, "trainer_state.json")
        if os.path.exists(spath):
            with open(spath) as f:
                out["state"] = json.load(f)
        opath = os.path.join(path, f"optimizer_state_rank{ctx.global_rank}.pt")
        if not os.path.exists(opath):
            # a checkpoint written by the reference, or by one process, has the one file only
            opath = os.path.join(path, "optimizer_state.pt")
        if os.path.exists(opath):
            sd = torch.load(opath, map_location="cpu", weights_only=False)
            why = self.optimizer.state_dict_mismatch(sd) if hasattr(self.optimizer, "state_dict_mismatch") else None
            st = out["state"]
            if why is None and st is not None and "trainer_step" in sd and sd["trainer_step"] != st.get("step_count"):
                why = (f"optimizer shard is of step {sd['trainer_step']}, trainer_state.json of step "
                       f"{st.get('step_count')} (a save was interrupted)")
            if why is None:
                out["opt"] = sd
            else:
                logger.warning("load_checkpoint(%s): optimizer state not restored: %s", path, why)
        return out

    def _all_ranks_have(self, flags: List[bool]) -> List[bool]:
        """Element-wise AND of ``flags`` over every rank of the job."""
        ctx = self.parallel_ctx
        if ctx.world_size <= 1 or not dist.is_initialized():
            return list(flags)
        t = torch.tensor([int(bool(f)) for f in flags], dtype=torch.int32, device=self.device)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        return [bool(v) for v in t.tolist()]

    def load_checkpoint(self, path: str) -> bool:
        """Tolerant restore: returns False instead of raising when files are absent or do not match; True when the
        optimizer state came back too.  Reading is local; what gets applied is agreed over all ranks first, because
        applying ends in collectives (re-publishing parameters from the restored masters): a part that one rank lacks
        (its optimizer shard is missing, of another layout or of another step) is skipped by every rank."""
        try:
            got = self._read_checkpoint(path)
            read_ok = True
        except Exception as e:  # noqa: BLE001 - restore is best-effort by contract
            logger.warning("load_checkpoint(%s) failed: %s", path, e)
            got, read_ok = {"weights": False, "lora": None, "opt": None, "state": None}, False
        read_ok, has_w, has_l, has_o = self._all_ranks_have(
            [read_ok, got["weights"], got["lora"] is not None, got["opt"] is not None])
        if not read_ok:
            return False
        if has_w:
            try:
                with self.optimizer.eval_mode():
                    load_from_hf_checkpoint(self.model, path)
                    self.optimizer.refresh_masters_from_params()
            except (ValueError, KeyError, OSError) as e:
                # every rank reads the same files and fails alike (the loader copies nothing unless all shapes fit)
                logger.warning("load_checkpoint(%s): weights not restored: %s", path, e)
                return False
        if has_l:
            load_lora_state_dict(self.model, got["lora"])
            self.optimizer.refresh_masters_from_params()
        ok = has_o and bool(self.optimizer.load_state_dict(got["opt"]))
        st = got["state"]
        if st is not None:
            self.step_count = int(st.get("step_count", 0))
            self.lr_scheduler.load_state_dict(st.get("lr_scheduler", {}))
        return ok

    # ---- reports ------------------------------------------------------------------------------------
    def generate_memory_report(self, batch_tokens: int = 0) -> MemoryReport:
        cfg, mc = self.config, self.model_config
        total = mc.num_params()
        trainable = sum(p.numel() for p in self.model.parameters() if p.requires_grad) * cfg.tp_size * cfg.pp_size \
            if cfg.lora_rank > 0 else total
        bd = MemoryBreakdown.estimate(total, trainable, 2 if self.dtype == torch.bfloat16 else 4, cfg.tp_size,
                                      cfg.pp_size, cfg.dp_size, cfg.zero_stage, batch_tokens, mc.hidden_size,
                                      mc.num_layers, mc.vocab_size, mc.intermediate_size,
                                      cfg.use_gradient_checkpoint)
        self.memory_profiler.snapshot("report")
        return MemoryReport.from_profiler(self.memory_profiler, bd, self.optimizer.memory_bytes())
