"""YAML configuration -> dataclasses, with the reference's key paths and validation.

Key paths are the ones ``scripts/run_colocate.py`` reads (scripts/run_colocate.py:187-262): ``model.*``,
``runtime.*``, ``distributed.*``, ``training.*``, ``lora.*``, ``rollout.*`` (``inference_preview.*`` in SFT
mode), ``data.*``, ``eval.*``, ``checkpoint.*``, ``experiment.*``, ``profiling.*``, ``icepop.*``,
``c3po_plus.*``, ``swift_sync.*``, ``async_pipeline.*``, ``vllm.*``.  ``training.zero_stage`` is the key that
counts (``distributed.zero_stage`` is accepted as a fallback: the reference silently ignores it, which
made its published "zero_stage 0" runs use stage 1).  CLI flags override YAML, YAML overrides defaults.
Unknown keys are reported instead of being silently dropped.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field, fields
from typing import Any, Dict, List, Optional, Tuple

import yaml


def load_yaml_config(path: Optional[str]) -> Dict[str, Any]:
    if not path:
        return {}
    with open(path) as f:
        return yaml.safe_load(f) or {}


def get_nested(d: Dict[str, Any], dotted: str, default=None):
    cur: Any = d
    for part in dotted.split("."):
        if not isinstance(cur, dict) or part not in cur:
            return default
        cur = cur[part]
    return cur


@dataclass
class ColocateConfig:
    model_path: str = "Qwen/Qwen3-0.6B"
    model_preset: Optional[str] = None      # random-init architecture instead of a checkpoint directory
    tp_size: int = 1
    pp_size: int = 1
    num_micro_batches: int = 1
    dp_size: int = 1
    sequence_parallel: bool = False
    max_seq_len: int = 2048
    use_flash_attn: bool = False
    attention_backend: str = "sdpa"
    use_gradient_checkpoint: bool = False
    training_mode: str = "grpo"
    output_dir: str = "outputs"
    checkpoint_save_dir: str = "checkpoints"
    checkpoint_save_interval: int = 0
    checkpoint_save_enabled: bool = True
    checkpoint_keep_last: int = 0           # > 0: only the newest N ``iter_*`` directories are kept (``latest`` / ``final`` always)
    resume_from: Optional[str] = None
    train_steps_per_iteration: int = 1
    total_iterations: int = 10
    lora_rank: int = 16
    lora_alpha: float = 32.0
    lora_target_modules: List[str] = field(default_factory=lambda: [
        "q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj"])
    learning_rate: float = 1e-5
    weight_decay: float = 0.01
    max_grad_norm: float = 1.0
    amp_dtype: str = "bf16"
    gradient_accumulation_steps: int = 4
    grpo_beta: float = 0.1
    grpo_clip_eps: float = 0.2
    lr_scheduler_type: str = "cosine"
    warmup_steps: int = 100
    min_lr_ratio: float = 0.1
    zero_stage: int = 1
    inference_backend: str = "vllm"         # "custom" / "native" (paged engine), "vllm", "mock"
    inference_preview_enabled: bool = True
    vllm_url: str = "http://localhost:8000"
    num_samples_per_prompt: int = 4
    max_tokens: int = 512
    temperature: float = 0.7
    top_p: float = 0.95
    sleep_level: int = 1
    ipc_chunk_size: int = 16
    batch_size: int = 4
    max_data_samples: int = 200
    dataset_name: str = "openai/gsm8k"
    dataset_config: Optional[str] = "main"
    dataset_split: str = "train"
    prompt_template: str = "qwen3_math"
    prompt_field: str = "question"
    input_field: Optional[str] = None
    response_field: str = "answer"
    answer_field: Optional[str] = "answer"
    eval_max_tokens: int = 128
    eval_num_prompts: int = 0
    memory_profile_interval: int = 100
    enable_profiling: bool = False
    profile_interval: int = 10
    enable_comm_overlap: bool = False
    reward_correct: float = 1.0            # reward.correct_reward: the answer is right
    reward_format: float = -0.5            # reward.format_reward: wrong or missing answer, well-formed response
    reward_wrong: float = -1.0             # reward.wrong_reward: wrong or missing answer, no recognisable format
    deterministic: bool = False            # fixed seeds, deterministic torch algorithms, no split-K atomics in the GEMM
    heartbeat_interval_s: float = 0.0      # > 0: ranks watch each other over the rendezvous store; a step is refused
    heartbeat_timeout_s: float = 10.0      # (PeerLostError ends the run) once a peer has been silent this long
    icepop_enabled: bool = False
    icepop_divergence_threshold: float = 0.5
    icepop_max_mask_ratio: float = 0.5
    c3po_plus_enabled: bool = False
    c3po_plus_token_budget: int = 1024
    c3po_plus_target_batch_tokens: int = 4096
    c3po_plus_packing_strategy: str = "ffd"
    swift_sync_enabled: bool = False
    swift_sync_fallback_full_every: int = 10
    swift_sync_double_buffer: bool = True
    async_pipeline_enabled: bool = False
    async_pipeline_max_staleness: int = 2
    async_pipeline_queue_size: int = 2
    max_retries: int = 3
    retry_delay: float = 2.0
    # ---- additions -----------------------------------------------------------------------------------
    synthetic_data: bool = False            # seeded random-token prompts + the synthetic token reward
    synthetic_prompt_len: int = 256
    synthetic_reward_dense_weight: float = 0.0   # > 0 adds a dense shaping term (non-zero advantages for a random policy)
    kv_cache_dtype: str = "fp16"
    kv_num_blocks: int = 0                  # 0: size from free memory
    enable_cuda_graph: bool = False
    use_radix_cache: bool = False
    seed: int = 0
    tensorboard: bool = True


# YAML path -> (field, section used in SFT mode instead, if any)
_YAML_MAP: List[Tuple[str, str]] = [
    ("model.name_or_path", "model_path"), ("model.preset", "model_preset"), ("model.max_seq_len", "max_seq_len"),
    ("model.use_flash_attn", "use_flash_attn"), ("model.attention_backend", "attention_backend"),
    ("model.use_gradient_checkpoint", "use_gradient_checkpoint"),
    ("runtime.tp_size", "tp_size"), ("runtime.dp_size", "dp_size"), ("runtime.precision", "amp_dtype"),
    ("runtime.inference_backend", "inference_backend"), ("runtime.enable_comm_overlap", "enable_comm_overlap"),
    ("runtime.sequence_parallel", "sequence_parallel"), ("runtime.seed", "seed"), ("runtime.deterministic", "deterministic"),
    ("runtime.heartbeat_interval_s", "heartbeat_interval_s"), ("runtime.heartbeat_timeout_s", "heartbeat_timeout_s"),
    ("reward.correct_reward", "reward_correct"), ("reward.format_reward", "reward_format"),
    ("reward.wrong_reward", "reward_wrong"),
    ("distributed.pp_size", "pp_size"), ("distributed.num_micro_batches", "num_micro_batches"),
    ("distributed.zero_stage", "zero_stage"),
    ("training.mode", "training_mode"), ("training.total_iterations", "total_iterations"),
    ("training.batch_size", "batch_size"), ("training.train_steps_per_iteration", "train_steps_per_iteration"),
    ("training.gradient_accumulation_steps", "gradient_accumulation_steps"),
    ("training.learning_rate", "learning_rate"), ("training.weight_decay", "weight_decay"),
    ("training.max_grad_norm", "max_grad_norm"), ("training.grpo_beta", "grpo_beta"),
    ("training.grpo_clip_eps", "grpo_clip_eps"), ("training.lr_scheduler", "lr_scheduler_type"),
    ("training.warmup_steps", "warmup_steps"), ("training.min_lr_ratio", "min_lr_ratio"),
    ("training.zero_stage", "zero_stage"),
    ("lora.rank", "lora_rank"), ("lora.alpha", "lora_alpha"), ("lora.target_modules", "lora_target_modules"),
    ("rollout.num_samples_per_prompt", "num_samples_per_prompt"), ("rollout.max_tokens", "max_tokens"),
    ("rollout.temperature", "temperature"), ("rollout.top_p", "top_p"),
    ("data.dataset_name", "dataset_name"), ("data.dataset_config", "dataset_config"), ("data.split", "dataset_split"),
    ("data.max_samples", "max_data_samples"), ("data.prompt_template", "prompt_template"),
    ("data.prompt_field", "prompt_field"), ("data.input_field", "input_field"),
    ("data.response_field", "response_field"), ("data.answer_field", "answer_field"),
    ("data.synthetic", "synthetic_data"), ("data.synthetic_prompt_len", "synthetic_prompt_len"),
    ("data.synthetic_reward_dense_weight", "synthetic_reward_dense_weight"),
    ("eval.max_tokens", "eval_max_tokens"), ("eval.num_prompts", "eval_num_prompts"),
    ("checkpoint.save_dir", "checkpoint_save_dir"), ("checkpoint.save_interval", "checkpoint_save_interval"),
    ("checkpoint.save_enabled", "checkpoint_save_enabled"), ("checkpoint.resume_from", "resume_from"),
    ("checkpoint.keep_last", "checkpoint_keep_last"),
    ("experiment.output_dir", "output_dir"),
    ("profiling.enabled", "enable_profiling"), ("profiling.interval", "profile_interval"),
    ("icepop.enabled", "icepop_enabled"), ("icepop.divergence_threshold", "icepop_divergence_threshold"),
    ("icepop.max_mask_ratio", "icepop_max_mask_ratio"),
    ("c3po_plus.enabled", "c3po_plus_enabled"), ("c3po_plus.token_budget", "c3po_plus_token_budget"),
    ("c3po_plus.target_batch_tokens", "c3po_plus_target_batch_tokens"),
    ("c3po_plus.packing_strategy", "c3po_plus_packing_strategy"),
    ("swift_sync.enabled", "swift_sync_enabled"), ("swift_sync.fallback_full_every", "swift_sync_fallback_full_every"),
    ("swift_sync.double_buffer", "swift_sync_double_buffer"),
    ("async_pipeline.enabled", "async_pipeline_enabled"), ("async_pipeline.max_staleness", "async_pipeline_max_staleness"),
    ("async_pipeline.queue_size", "async_pipeline_queue_size"),
    ("vllm.url", "vllm_url"),
    ("inference.kv_cache_dtype", "kv_cache_dtype"), ("inference.num_blocks", "kv_num_blocks"),
    ("inference.enable_cuda_graph", "enable_cuda_graph"), ("inference.use_radix_cache", "use_radix_cache"),
]
# keys present in the reference's YAML files that no code reads; accepted silently
# keys of the reference's YAML files that neither it nor this framework acts on (accepted silently)
_DOCUMENTATION_ONLY = {"lora.dropout", "lora.enabled", "experiment.name", "experiment.seed", "experiment.stage",
                       "experiment.algorithm", "profiling.memory", "profiling.comm", "profiling.compute",
                       "profiling.compute_mfu", "profiling.memory_breakdown", "profiling.metrics",
                       "profiling.track_communication", "reward.type", "reward.answer_format", "runtime.device",
                       "model.trust_remote_code", "model.sft_checkpoint", "icepop.log_diagnostics"}


def _flatten(d: Dict[str, Any], prefix: str = "") -> Dict[str, Any]:
    out = {}
    for k, v in d.items():
        key = f"{prefix}{k}"
        if isinstance(v, dict):
            out.update(_flatten(v, key + "."))
        else:
            out[key] = v
    return out


_BOOL_WORDS = {"true": True, "yes": True, "on": True, "1": True, "false": False, "no": False, "off": False, "0": False}


def _coerce(value, kind: str, where: str):
    """Bring a YAML / command-line value to the type of its field (named by the dataclass annotation).  YAML reads
    ``1e-5`` (no dot) as a string and ``2.0`` as a float: both are what the user meant for a float / an int field, so
    they are converted; anything that does not convert raises ``ValueError`` naming the key."""
    kind = kind.replace("Optional[", "").rstrip("]") if kind.startswith("Optional[") else kind
    try:
        if kind == "float" and not isinstance(value, bool):
            if isinstance(value, (int, float, str)):
                return float(value)
        elif kind == "int" and not isinstance(value, bool):
            if isinstance(value, int):
                return value
            f = float(value)
            if f == int(f):
                return int(f)
            raise ValueError("not a whole number")
        elif kind == "bool":
            if isinstance(value, bool):
                return value
            if isinstance(value, (int, str)) and str(value).strip().lower() in _BOOL_WORDS:
                return _BOOL_WORDS[str(value).strip().lower()]
        elif kind == "str":
            if isinstance(value, (str, int, float)) and not isinstance(value, bool):
                return str(value)
        elif kind.startswith("List["):
            if isinstance(value, (list, tuple)):
                return list(value)
            if isinstance(value, str):
                return [v.strip() for v in value.split(",") if v.strip()]
        else:
            return value                        # a type this function does not know: leave it to the consumer
    except (TypeError, ValueError) as e:
        raise ValueError(f"{where}: {value!r} is not a valid {kind} ({e})") from None
    raise ValueError(f"{where}: {value!r} is not a valid {kind}")


def _field_kinds(cls) -> Dict[str, str]:
    import dataclasses
    return {f.name: (f.type if isinstance(f.type, str) else getattr(f.type, "__name__", str(f.type)))
            for f in dataclasses.fields(cls)}


def build_colocate_config(yaml_cfg: Dict[str, Any], overrides: Optional[Dict[str, Any]] = None
                          ) -> Tuple[ColocateConfig, List[str]]:
    """Returns the config and the list of YAML keys that were not understood."""
    cfg = ColocateConfig()
    kinds = _field_kinds(ColocateConfig)
    known = {p for p, _ in _YAML_MAP}
    mode = get_nested(yaml_cfg, "training.mode", cfg.training_mode)
    for path, name in _YAML_MAP:
        if path == "distributed.zero_stage" and get_nested(yaml_cfg, "training.zero_stage") is not None:
            continue
        v = get_nested(yaml_cfg, path)
        if v is not None:
            setattr(cfg, name, _coerce(v, kinds.get(name, ""), path))
    for key, name in (("max_tokens", "max_tokens"), ("temperature", "temperature"), ("top_p", "top_p"),
                      ("enabled", "inference_preview_enabled")):
        known.add(f"inference_preview.{key}")
        v = get_nested(yaml_cfg, f"inference_preview.{key}")
        # SFT previews read their sampling knobs from inference_preview.*; GRPO reads rollout.*
        if v is not None and (mode == "sft" or key == "enabled"):
            setattr(cfg, name, _coerce(v, kinds.get(name, ""), f"inference_preview.{key}"))
    for k, v in (overrides or {}).items():
        if v is not None:
            if not hasattr(cfg, k):
                raise KeyError(f"unknown override {k!r}")
            setattr(cfg, k, _coerce(v, kinds.get(k, ""), f"override {k}"))
    unknown = sorted(k for k in _flatten(yaml_cfg) if k not in known and k not in _DOCUMENTATION_ONLY)
    return cfg, unknown


def validate_parallel_config(cfg: ColocateConfig, world_size: Optional[int] = None) -> None:
    """The reference's checks (scripts/run_colocate.py:86-136), raising ValueError with the reason."""
    world = world_size if world_size is not None else int(os.environ.get("WORLD_SIZE", "1"))
    for name, least in (("pp_size", 1), ("tp_size", 1), ("dp_size", 1), ("num_micro_batches", 1), ("batch_size", 1),
                        ("gradient_accumulation_steps", 1), ("max_seq_len", 2), ("lora_rank", 0), ("zero_stage", 0)):
        v = getattr(cfg, name, least)
        if not isinstance(v, int) or isinstance(v, bool) or v < least:
            raise ValueError(f"{name} must be an integer >= {least}, not {v!r}")
    if not cfg.learning_rate >= 0 or cfg.learning_rate == float("inf"):
        raise ValueError(f"learning_rate must be a finite number >= 0, not {cfg.learning_rate!r}")
    if cfg.zero_stage > 3:
        raise ValueError(f"zero_stage must be 0, 1, 2 or 3, not {cfg.zero_stage}")
    if cfg.pp_size * cfg.tp_size * cfg.dp_size != world:
        raise ValueError(f"pp({cfg.pp_size}) * tp({cfg.tp_size}) * dp({cfg.dp_size}) != WORLD_SIZE({world})")
    if cfg.num_micro_batches < cfg.pp_size:
        raise ValueError(f"num_micro_batches({cfg.num_micro_batches}) must be >= pp_size({cfg.pp_size})")
    if cfg.batch_size % (cfg.num_micro_batches * cfg.dp_size) != 0:
        raise ValueError(f"batch_size({cfg.batch_size}) must be divisible by num_micro_batches*dp_size "
                         f"({cfg.num_micro_batches}*{cfg.dp_size})")
    if cfg.pp_size > 1 and cfg.zero_stage > 1:
        raise ValueError("pipeline parallelism requires zero_stage <= 1")
    if cfg.pp_size > 1 and cfg.training_mode != "sft":
        raise ValueError("pipeline parallelism supports training.mode == sft only")
    if cfg.amp_dtype not in ("fp32", "bf16", "fp16"):
        raise ValueError(f"runtime.precision must be fp32, bf16 or fp16, not {cfg.amp_dtype!r}")
    if cfg.training_mode not in ("grpo", "sft"):
        raise ValueError(f"training.mode must be grpo or sft, not {cfg.training_mode!r}")


def config_snapshot(cfg) -> Dict[str, Any]:
    return {f.name: getattr(cfg, f.name) for f in fields(cfg)}


def apply_determinism(enabled: bool, seed: int = 0) -> None:
    """``runtime.deterministic`` (scripts/run_colocate.py:144-170 of the reference).  On: seed Python / NumPy / torch,
    ask torch for deterministic algorithms (warn only), fix cuDNN's choices, and set ``B200FW_DETERMINISTIC=1`` so the
    GEMM keeps one unit per output tile instead of split-K slices that add with float atomics.  What stays
    order-dependent in fp32: the loss sum, the norm weight-gradient and embedding-gradient accumulations (float
    atomics inside those kernels) - runs then agree to summation-order rounding, not bit for bit.  Off: the switches
    are cleared, so a previous setting in the process or its environment does not linger."""
    import os
    import random

    import torch
    if enabled:
        os.environ["B200FW_DETERMINISTIC"] = "1"
        os.environ.setdefault("CUBLAS_WORKSPACE_CONFIG", ":4096:8")
        random.seed(seed)
        try:
            import numpy as np
            np.random.seed(seed % (1 << 32))
        except ImportError:
            pass
        torch.manual_seed(seed)
        torch.use_deterministic_algorithms(True, warn_only=True)
        torch.backends.cudnn.deterministic, torch.backends.cudnn.benchmark = True, False
    else:
        os.environ.pop("B200FW_DETERMINISTIC", None)
        torch.use_deterministic_algorithms(False)
        torch.backends.cudnn.deterministic, torch.backends.cudnn.benchmark = False, True

