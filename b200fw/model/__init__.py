"""Qwen3-style decoder with tensor / sequence / pipeline parallel layers, LoRA and HF checkpoint IO."""
from .config import ModelConfig, PRESETS
from .qwen3 import (
    RMSNorm, ColumnParallelLinear, RowParallelLinear, ParallelMLP, ParallelAttention,
    ParallelTransformerLayer, ParallelTransformerModel,
)
from .hf_io import load_from_hf_checkpoint, save_hf_checkpoint, write_hf_config, read_hf_config
from .lora import (LoRALayer, LoRAColumnParallel, LoRARowParallel, LinearWithLoRA, apply_lora,
                   merge_lora_weights, get_lora_state_dict)

__all__ = [
    "ModelConfig", "PRESETS", "RMSNorm", "ColumnParallelLinear", "RowParallelLinear", "ParallelMLP",
    "ParallelAttention", "ParallelTransformerLayer", "ParallelTransformerModel",
    "load_from_hf_checkpoint", "save_hf_checkpoint", "write_hf_config", "read_hf_config",
    "LoRALayer", "LoRAColumnParallel", "LoRARowParallel", "LinearWithLoRA", "apply_lora",
    "merge_lora_weights", "get_lora_state_dict",
]
