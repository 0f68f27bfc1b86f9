"""TrainWorker / InferWorker: the two roles of disaggregated training behind the reference's worker API.

In the reference these are Ray actors (``@ray.remote(num_gpus=2)``) created lazily so that importing the
module does not need Ray (src/engines/train_worker.py:24-160, src/engines/infer_worker.py:25-323).  Here they
are plain classes that run inside the rank that owns the role - the disaggregated orchestrator splits one
``torchrun`` world into trainer ranks and rollout ranks - and ``get_train_worker_class()`` /
``get_infer_worker_class()`` wrap them with ``ray.remote`` only when Ray is importable.

Differences, on purpose: ``InferWorker.update_weights(mode="full")`` really copies the tensors into the live
engine (the reference's custom backend only invalidates caches); ``mode="delta"`` keeps the reference's
double-buffered adapter state and, when the worker was given a ``merge_fn``, re-merges the active adapters
into the engine's weights; prompts may be strings (tokenizer needed) or token-id lists (answers are then
token-id lists too).
"""
from __future__ import annotations

import time
from typing import Callable, Dict, List, Optional, Sequence, Union

import torch

from ..infer import InferenceConfig, InferenceEngine
from ..obs.logging import get_logger
from ..sync.double_buffer import DoubleBufferedLoRA
from ..train.engine import TrainConfig, TrainEngine, TrainMetrics

logger = get_logger("workers")

__all__ = ["TrainWorker", "InferWorker", "get_train_worker_class", "get_infer_worker_class"]


def _gpu_status(peak: bool) -> Optional[dict]:
    if not torch.cuda.is_available():
        return None
    d = torch.cuda.current_device()
    out = {"device_id": d, "allocated_mb": torch.cuda.memory_allocated(d) / 2 ** 20,
           "reserved_mb": torch.cuda.memory_reserved(d) / 2 ** 20}
    if peak:
        out["peak_mb"] = torch.cuda.max_memory_allocated(d) / 2 ** 20
    return out


class TrainWorker:
    """Owns a :class:`TrainEngine`; every call but the constructor requires ``initialize()`` first."""

    def __init__(self, config: TrainConfig, engine_factory: Optional[Callable[[TrainConfig], TrainEngine]] = None):
        self.config = config
        self.engine: Optional[TrainEngine] = None
        self._factory = engine_factory or TrainEngine
        self._initialized = False
        self._step_count = 0
        self._total_train_time = 0.0

    def initialize(self) -> bool:
        self.engine = self._factory(self.config)
        self.engine.initialize()
        self._initialized = True
        return True

    def _need(self):
        assert self._initialized, "TrainWorker not initialized. Call initialize() first."

    def train_step(self, prompts_tokens: List[List[int]], responses_group: List[List[List[int]]],
                   rewards_group: List[List[float]], **kw) -> TrainMetrics:
        """One GRPO step on ``B`` prompts with ``K`` responses each (extra keywords go to ``grpo_step``)."""
        self._need()
        t0 = time.perf_counter()
        m = self.engine.grpo_step(prompts_tokens=prompts_tokens, responses_group=responses_group,
                                  rewards_group=rewards_group, **kw)
        self._total_train_time += time.perf_counter() - t0
        self._step_count += 1
        return m

    def sft_step(self, prompts_tokens: List[List[int]], response_tokens: List[List[int]]) -> TrainMetrics:
        self._need()
        t0 = time.perf_counter()
        m = self.engine.sft_step(prompts_tokens, response_tokens)
        self._total_train_time += time.perf_counter() - t0
        self._step_count += 1
        return m

    def export_weights(self, device: Optional[str] = None) -> Dict[str, torch.Tensor]:
        """Merged (LoRA folded in) weights under their HF names."""
        self._need()
        return self.engine.export_weights(device)

    def export_lora_delta(self) -> Dict[str, torch.Tensor]:
        self._need()
        return self.engine.export_lora_delta()

    def save_checkpoint(self, path: str):
        self._need()
        self.engine.save_checkpoint(path)

    def load_checkpoint(self, path: str) -> bool:
        self._need()
        return self.engine.load_checkpoint(path)

    def get_status(self) -> dict:
        c = self.config
        status = {"initialized": self._initialized, "step_count": self._step_count,
                  "total_train_time_s": self._total_train_time,
                  "config": {"model_path": c.model_path, "tp_size": c.tp_size, "lora_rank": c.lora_rank}}
        gpu = _gpu_status(peak=True)
        if gpu is not None:
            status["gpu"] = gpu
        if self._initialized and self.engine is not None and self.engine.model is not None:
            ps = list(self.engine.model.parameters())
            status["trainable_params"] = sum(p.numel() for p in ps if p.requires_grad)
            status["total_params"] = sum(p.numel() for p in ps)
        return status


Prompt = Union[str, Sequence[int]]


class InferWorker:
    """Owns a rollout :class:`InferenceEngine`.

    ``model`` (a built ``ParallelTransformerModel``) or ``model_path`` (HF directory) selects the paged
    ``kv_cache`` engine; with neither the engine runs in ``mock`` mode (scheduler + random tokens), which
    is what the reference's custom backend always does.  ``backend="vllm"`` builds an in-process ``vllm.LLM`` on
    ``model_path`` as the reference does (src/engines/infer_worker.py:90-99,139-162): a library engine, kept for
    parity; it needs a real HF model directory and takes text (or token-id) prompts.  Weight updates reach it through
    ``VLLMClient`` / ``IPCWeightTransfer`` against a server, not through this class.
    """

    def __init__(self, model_path: Optional[str] = None, tp_size: int = 1, gpu_memory_utilization: float = 0.85,
                 max_model_len: int = 4096, backend: str = "custom", inference_config: Optional[InferenceConfig] = None,
                 model=None, tokenizer=None, merge_fn: Optional[Callable[[Dict[str, torch.Tensor]], Dict[str, torch.Tensor]]] = None):
        if backend not in ("custom", "mock", "vllm"):
            raise ValueError(f"InferWorker backend {backend!r}: expected 'custom' (native engine), 'mock' or 'vllm'")
        if backend == "vllm" and not model_path:
            raise ValueError("InferWorker backend 'vllm' needs model_path (a Hugging Face model directory)")
        self.model_path, self.tp_size = model_path, tp_size
        self.gpu_memory_utilization, self.max_model_len, self.backend = gpu_memory_utilization, max_model_len, backend
        self._config, self._model, self._tokenizer, self._merge_fn = inference_config, model, tokenizer, merge_fn
        self._engine: Optional[InferenceEngine] = None
        self._double_buffer: Optional[DoubleBufferedLoRA] = None
        self._initialized = False
        self._total_generate_time = 0.0
        self._total_requests = 0
        self._weight_version = 0

    # ---- lifecycle ------------------------------------------------------------------------------------
    def initialize(self) -> bool:
        if self.backend == "vllm":
            try:
                from vllm import LLM
            except Exception as e:  # noqa: BLE001
                raise RuntimeError(f"InferWorker backend 'vllm': the vllm package cannot be imported ({e})") from e
            self._vllm = LLM(model=self.model_path, tensor_parallel_size=self.tp_size,
                             gpu_memory_utilization=self.gpu_memory_utilization, max_model_len=self.max_model_len,
                             trust_remote_code=True)
            self._initialized = True
            return True
        cfg = self._config
        if cfg is None:
            have_model = self._model is not None or (self.model_path is not None and self.backend != "mock")
            cfg = InferenceConfig(max_num_batched_tokens=2048, max_num_sequences=256, enable_prefix_caching=True,
                                  inference_mode="kv_cache" if have_model else "mock")
            if self.model_path is not None and have_model:
                cfg.model_path = self.model_path
            if self._model is not None:
                cfg = InferenceConfig.from_model_config(self._model.cfg, **{
                    k: getattr(cfg, k) for k in ("max_num_batched_tokens", "max_num_sequences", "enable_prefix_caching",
                                                 "inference_mode")})
        self._engine = InferenceEngine(cfg, model=self._model) if self._model is not None else InferenceEngine(cfg)
        self._engine.initialize()
        self._initialized = True
        return True

    @property
    def engine(self) -> Optional[InferenceEngine]:
        return self._engine

    def _tok(self):
        if self._tokenizer is None:
            from ..data.pipeline import _load_tokenizer
            self._tokenizer = _load_tokenizer(self.model_path)
        return self._tokenizer

    # ---- generation -----------------------------------------------------------------------------------
    def generate(self, prompts: List[Prompt], num_samples: int = 4, max_tokens: int = 512,
                 temperature: float = 0.7, top_p: Optional[float] = None) -> List[List]:
        """``[num_prompts][num_samples]`` answers: text for text prompts, token ids for token-id prompts.
        All ``num_prompts * num_samples`` requests go to the engine as one batch (the samples of a prompt
        share its prefix blocks); a request dropped by an out-of-memory recovery yields ``""`` / ``[]``."""
        assert self._initialized, "InferWorker not initialized. Call initialize() first."
        t0 = time.perf_counter()
        as_text = [isinstance(p, str) for p in prompts]
        if self.backend == "vllm":
            from vllm import SamplingParams
            sp = SamplingParams(n=num_samples, max_tokens=max_tokens, temperature=temperature,
                                top_p=0.95 if top_p is None else top_p)
            inputs = [p if t else {"prompt_token_ids": list(p)} for p, t in zip(prompts, as_text)]
            outs = self._vllm.generate(inputs, sp)
            results = [[(c.text if t else list(c.token_ids)) for c in o.outputs] for o, t in zip(outs, as_text)]
            self._total_generate_time += time.perf_counter() - t0
            self._total_requests += len(prompts)
            return results
        toks = [list(self._tok().encode(p)) if t else list(p) for p, t in zip(prompts, as_text)]
        batch = [t for t in toks for _ in range(num_samples)]
        outs = self._engine.generate(batch, max_tokens=max_tokens, temperature=temperature, top_p=top_p) if batch else []
        results: List[List] = []
        for i, text in enumerate(as_text):
            group = []
            for o in outs[i * num_samples:(i + 1) * num_samples]:
                if text:
                    group.append(self._tok().decode(o, skip_special_tokens=True) if o else "")
                else:
                    group.append(list(o) if o else [])
            results.append(group)
        self._total_generate_time += time.perf_counter() - t0
        self._total_requests += len(prompts)
        return results

    # ---- weights --------------------------------------------------------------------------------------
    def update_weights(self, state_dict: Dict[str, torch.Tensor], mode: str = "full") -> bool:
        """``mode="full"``: HF-named tensors copied into the live engine.  ``mode="delta"``: adapter deltas
        added to the shadow buffer, buffers swapped (the first call seeds the buffers with the full adapter
        state); with a ``merge_fn`` the active adapter state is merged and loaded too.  Returns ``False``
        (and leaves the version alone) on any failure."""
        assert self._initialized, "InferWorker not initialized."
        if self.backend == "vllm":
            logger.error("InferWorker backend 'vllm' takes weight updates through VLLMClient / IPCWeightTransfer")
            return False
        try:
            if mode == "delta":
                if self._double_buffer is None:
                    self._double_buffer = DoubleBufferedLoRA(state_dict)
                else:
                    self._double_buffer.apply_delta_to_shadow(state_dict)
                    self._double_buffer.swap_buffers()
                if self._merge_fn is not None and self._engine.model is not None:
                    self._engine.load_weights(self._merge_fn(self._double_buffer.get_active_state()))
                else:
                    self._engine.on_weights_updated()
            elif mode == "full":
                if getattr(self._engine, "model", None) is not None:
                    self._engine.load_weights(state_dict)
                else:
                    self._engine.on_weights_updated()
            else:
                raise ValueError(f"unknown weight update mode {mode!r}")
            self._weight_version += 1
            return True
        except Exception as e:  # noqa: BLE001 - the caller decides what a failed sync means
            logger.error("weight update failed: %s", e)
            return False

    # ---- status ---------------------------------------------------------------------------------------
    def health_check(self) -> bool:
        if self.backend == "vllm":
            return self._initialized and getattr(self, "_vllm", None) is not None
        return self._initialized and self._engine is not None and self._engine.initialized

    def get_status(self) -> dict:
        status = {"initialized": self._initialized, "backend": self.backend, "model_path": self.model_path,
                  "tp_size": self.tp_size, "weight_version": self._weight_version,
                  "total_requests": self._total_requests, "total_generate_time_s": self._total_generate_time}
        if self._engine is not None:
            status["engine_stats"] = self._engine.get_stats()
        if self._double_buffer is not None:
            status["lora_buffer_version"] = self._double_buffer.get_version()
        gpu = _gpu_status(peak=False)
        if gpu is not None:
            status["gpu"] = gpu
        return status


def _maybe_remote(cls, num_gpus: int):
    try:
        import ray
    except Exception:  # noqa: BLE001 - Ray is optional
        return cls
    return ray.remote(num_gpus=num_gpus)(cls)


def get_train_worker_class(num_gpus: int = 1):
    """``ray.remote(TrainWorker)`` when Ray is installed, else the plain class (same methods)."""
    return _maybe_remote(TrainWorker, num_gpus)


def get_infer_worker_class(num_gpus: int = 1):
    return _maybe_remote(InferWorker, num_gpus)
