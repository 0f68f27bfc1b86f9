"""Reward functions: the GSM8K rule reward and the synthetic token-rule reward used by the benchmarks."""
from .gsm8k import GSM8KRewardFunction, extract_answer, check_format
from .synthetic import SyntheticTokenReward

__all__ = ["GSM8KRewardFunction", "extract_answer", "check_format", "SyntheticTokenReward"]
