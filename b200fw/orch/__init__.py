"""Orchestration: the colocate loop (train and rollout on the same GPUs) and the disaggregated loop
(trainer rank group + rollout rank group in one world)."""
from .colocate import ColocateOrchestrator, IterationMetrics, OrchestratorState
from .disagg import DisaggConfig, DisaggOrchestrator
from .workers import InferWorker, TrainWorker, get_infer_worker_class, get_train_worker_class

__all__ = ["ColocateOrchestrator", "IterationMetrics", "OrchestratorState", "DisaggConfig", "DisaggOrchestrator",
           "TrainWorker", "InferWorker", "get_train_worker_class", "get_infer_worker_class"]
