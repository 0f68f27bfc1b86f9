"""Observability: logging, metrics, memory, profilers, timeline and run artefacts."""
from .logging import setup_logger, get_logger
from .metrics import MetricsCollector
from .artifacts import ArtifactWriter
from .memory import MemoryProfiler, MemoryBreakdown, MemoryReport, MemoryManager
from .profilers import CommProfiler, ComputeProfiler
from .timeline import ScheduleVisualizer
from . import nvtx
from .tb_events import EventFileWriter, read_scalars, open_writer
from .eval_utils import EvalMetrics, compute_token_f1, compute_bleu4, compute_exact_match, normalize_text

__all__ = [
    "setup_logger", "get_logger", "MetricsCollector", "ArtifactWriter", "MemoryProfiler", "MemoryBreakdown",
    "MemoryReport", "MemoryManager", "CommProfiler", "ComputeProfiler", "ScheduleVisualizer", "EvalMetrics",
    "compute_token_f1", "compute_bleu4", "compute_exact_match", "normalize_text", "EventFileWriter", "read_scalars",
    "open_writer", "nvtx",
]
