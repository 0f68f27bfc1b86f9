"""Training engine (SFT + GRPO), IcePop train/infer divergence filter, C3PO++ rollout chunking."""
from .engine import TrainConfig, TrainMetrics, TrainEngine
from .icepop import IcePopConfig, IcePopFilter
from .c3po import C3POConfig, ResponseChunk, C3POPlusScheduler

__all__ = ["TrainConfig", "TrainMetrics", "TrainEngine", "IcePopConfig", "IcePopFilter", "C3POConfig",
           "ResponseChunk", "C3POPlusScheduler"]
