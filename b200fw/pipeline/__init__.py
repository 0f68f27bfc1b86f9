"""Pipeline parallelism: layer -> stage split and the 1F1B schedule over NCCL / gloo p2p."""
from .stages import split_layers_to_stages, PipelineParallelContext
from .schedule_1f1b import PipelineScheduler

__all__ = ["split_layers_to_stages", "PipelineParallelContext", "PipelineScheduler"]
