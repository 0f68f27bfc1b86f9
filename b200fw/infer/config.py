"""InferenceConfig: the reference's field set (src/inference/engine.py:60-194) plus the native engine's
own knobs."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch


@dataclass
class InferenceConfig:
    num_layers: int = 32
    num_heads: int = 32
    num_kv_heads: int = 8
    head_dim: int = 128
    hidden_size: int = 4096
    vocab_size: int = 151936
    num_blocks: int = 1024
    block_size: int = 16
    kv_cache_dtype: str = "fp16"        # "fp16" (16-bit, in the model's dtype) or "fp8" (e4m3 + per-block scale)
    max_num_batched_tokens: int = 2048
    max_num_sequences: int = 256
    max_prefill_tokens: int = 1024
    enable_chunked_prefill: bool = True
    chunk_size: int = 512
    enable_prefix_caching: bool = False
    enable_cuda_graph: bool = False
    max_cached_blocks: int = 512
    enable_prefix_reuse: bool = True
    enable_async_scheduling: bool = False
    enable_partitioned_attention: bool = False
    attention_partition_size: int = 512
    use_radix_cache: bool = False
    radix_cache_max_nodes: int = 10000
    temperature: float = 0.7
    top_p: float = 0.9
    speculative_enabled: bool = False
    speculative_draft_model_path: str = ""
    speculative_num_tokens: int = 5
    inference_mode: str = "mock"         # "kv_cache" (native paged model) | "eager" (full recompute) | "mock"
    use_real_model: bool = False
    model_path: str = ""
    dtype: str = "bfloat16"
    # ---- additions ---------------------------------------------------------------------------------
    intermediate_size: int = 0
    eos_token_id: Optional[int] = None   # the reference hard-codes 2 (src/inference/scheduler.py:96-98)
    seed: int = 0
    speculative_draft_layers: int = 2    # random-init draft model of the same width when no path is given
    adaptive_chunking: bool = True
    # a weight update does not abort running requests: they go on under the new weights and keep the K/V their
    # earlier tokens produced under the old ones, for at most this many versions (0 = abort on every update)
    max_weight_staleness: int = 1
    # decode-only steps leave the sampled ids on the device: the next step's forward is launched from them before the
    # host has read them (one step late), so host-side scheduling overlaps the GPU's work.  The cost is one discarded
    # token after an EOS.  Turned off with speculative decoding (which needs the values every round).
    async_decode: bool = True
    # split every sequence's keys over a few CTAs when one CTA per (sequence, kv head) would fill only a few waves
    decode_balance_splits: bool = False

    @classmethod
    def from_model_config(cls, mc, **kw) -> "InferenceConfig":
        return cls(num_layers=mc.num_layers, num_heads=mc.num_heads, num_kv_heads=mc.num_kv_heads,
                   head_dim=mc.head_dim, hidden_size=mc.hidden_size, vocab_size=mc.vocab_size,
                   intermediate_size=mc.intermediate_size, **kw)

    def kv_bytes_per_block(self) -> int:
        el = 1 if self.kv_cache_dtype == "fp8" else 2
        return 2 * self.num_layers * self.block_size * self.num_kv_heads * self.head_dim * el

    @classmethod
    def auto_from_device(cls, num_layers=32, num_kv_heads=8, head_dim=128, block_size=16,
                         gpu_memory_fraction=0.3, max_blocks: int = 1 << 20, **kw) -> "InferenceConfig":
        """Size the block pool from free device memory (a fraction of it); CPU gets a small pool."""
        base = dict(num_layers=num_layers, num_kv_heads=num_kv_heads, head_dim=head_dim, block_size=block_size)
        if not torch.cuda.is_available():
            return cls(num_blocks=64, enable_cuda_graph=False, **base, **kw)
        try:
            free, total = torch.cuda.mem_get_info()
        except (RuntimeError, AssertionError):
            return cls(num_blocks=64, enable_cuda_graph=False, **base, **kw)
        probe = cls(**base, **{k: v for k, v in kw.items() if k == "kv_cache_dtype"})
        blocks = max(32, int(free * gpu_memory_fraction) // probe.kv_bytes_per_block())
        kw.setdefault("enable_cuda_graph", total > 12 * 1024 ** 3)
        return cls(num_blocks=min(blocks, max_blocks), **base, **kw)
