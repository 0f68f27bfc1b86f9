"""Optimizers: bucketed flat-buffer AdamW with ZeRO stage 0/1/2/3 sharding and LR schedules."""
from .schedule import LRSchedule
from .zero import ZeROOptimizer, ZeROStage2Optimizer, ZeROStage3Optimizer, build_optimizer

__all__ = ["LRSchedule", "ZeROOptimizer", "ZeROStage2Optimizer", "ZeROStage3Optimizer", "build_optimizer"]
