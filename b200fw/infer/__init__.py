"""Inference runtime: paged KV cache, continuous batching, prefix / radix cache, native model runner,
CUDA-graph decode, speculative decoding and the engine that ties them together."""
from .config import InferenceConfig
from .attention import PagedAttention, PartitionedPagedAttention, store_kv_cache
from .context import InferenceContext, get_context, reset_context, set_context
from .engine import InferenceEngine
from .graphs import CUDAGraphRunner
from .kv_cache import Block, BlockPool, BlockTable, KVCacheManager
from .prefix_cache import PrefixCache
from .radix_cache import RadixAttentionCache
from .runner import ModelRunner, ModelRunnerConfig
from .scheduler import ContinuousBatchingScheduler, Request, RequestState, SchedulerOutput
from .spec import SpeculativeConfig, SpeculativeDecoder, verify_greedy, verify_sampling

__all__ = [
    "InferenceConfig", "InferenceContext", "InferenceEngine", "CUDAGraphRunner", "Block", "BlockPool",
    "BlockTable", "KVCacheManager", "PrefixCache", "RadixAttentionCache", "ModelRunner",
    "ContinuousBatchingScheduler", "Request", "RequestState", "SchedulerOutput", "SpeculativeDecoder",
    "verify_greedy", "verify_sampling", "PagedAttention", "PartitionedPagedAttention", "store_kv_cache", "get_context",
    "set_context", "reset_context", "ModelRunnerConfig", "SpeculativeConfig",
]
