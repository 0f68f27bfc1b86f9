"""Reward functions: the GSM8K rule reward and the synthetic token-rule reward used by the benchmarks."""
from .gsm8k import GSM8KRewardFunction, check_format, compute_batch_rewards, compute_reward, extract_answer
from .synthetic import SyntheticTokenReward

__all__ = ["GSM8KRewardFunction", "extract_answer", "check_format", "SyntheticTokenReward", "compute_reward",
           "compute_batch_rewards"]
