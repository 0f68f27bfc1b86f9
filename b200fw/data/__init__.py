"""Data pipelines: GSM8K-style prompt/answer batches and the seeded synthetic token dataset."""
from .pipeline import GRPOBatch, GSM8KDataPipeline, SyntheticTokenPipeline, PROMPT_TEMPLATES, SimpleTokenizer

__all__ = ["GRPOBatch", "GSM8KDataPipeline", "SyntheticTokenPipeline", "PROMPT_TEMPLATES", "SimpleTokenizer"]
