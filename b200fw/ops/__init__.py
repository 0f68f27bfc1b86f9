"""Operators.  Every op has two implementations selected by the input's device:

* CUDA tensors run the hand-written sm_100a kernels from ``csrc/`` (there is no PyTorch fallback on a
  GPU: a missing kernel library raises);
* CPU tensors run a plain PyTorch fp32-accurate implementation, which is the numerical oracle of the
  test-suite and the path used by the gloo plumbing tests.
"""
from .gemm import gemm, linear, lora_linear, grad_into_main
from .elementwise import rmsnorm, qknorm_rope, qknorm_rope_store, swiglu, embedding, rope_tables
from .attention import flash_attention
from .loss import lm_head_cross_entropy, lm_head_logprob, grpo_token_loss, VocabShard, valid_rows
from .optim import sumsq, fused_adamw
from .paged import (kv_store, kv_gather, paged_decode_attention, paged_prefill_attention, varlen_attention,
                    topp_sample)

__all__ = [
    "gemm", "linear", "lora_linear", "grad_into_main", "rmsnorm", "qknorm_rope", "qknorm_rope_store", "swiglu", "embedding", "rope_tables",
    "flash_attention", "VocabShard", "valid_rows", "lm_head_cross_entropy", "lm_head_logprob", "grpo_token_loss", "sumsq",
    "fused_adamw", "kv_store", "kv_gather", "paged_decode_attention", "paged_prefill_attention", "varlen_attention", "topp_sample",
]
