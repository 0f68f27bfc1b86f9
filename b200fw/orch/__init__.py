"""Orchestration: the colocate loop (train and rollout on the same GPUs) and the disaggregated loop
(trainer rank group + rollout rank group in one world)."""
from .colocate import ColocateOrchestrator, IterationMetrics, OrchestratorState
from .disagg import DisaggConfig, DisaggOrchestrator

__all__ = ["ColocateOrchestrator", "IterationMetrics", "OrchestratorState", "DisaggConfig", "DisaggOrchestrator"]
