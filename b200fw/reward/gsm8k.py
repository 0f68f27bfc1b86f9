"""Rule-based GSM8K reward (behaviour of src/reward/gsm8k_reward.py:17-223).

Answer extraction tries, in order: ``#### <number>``, ``\\boxed{...}``, "the answer is" / "答案是" phrases,
then the last number in the text.  Reward: +1 for a correct answer; a wrong or missing answer gets -0.5 when
the response is well formed (step markers, several lines or an explicit answer marker) and -1 otherwise.
Running accuracy statistics are kept.
"""
from __future__ import annotations

import re
from typing import Dict, List, Optional

_NUM = r"-?\d[\d,]*(?:\.\d+)?(?:/\d+)?"
_PATTERNS = [
    re.compile(r"####\s*\$?\s*(" + _NUM + ")"),
    re.compile(r"\\boxed\{\s*\$?\s*(" + _NUM + r")\s*\}"),
    re.compile(r"(?:final answer|answer)\s*(?:is|:|=)\s*\$?\s*(" + _NUM + ")", re.IGNORECASE),
    re.compile(r"(?:答案是|答案为|答案[:：])\s*\$?\s*(" + _NUM + ")"),
]
_LAST = re.compile(_NUM)


def _to_float(s: str) -> Optional[float]:
    s = s.replace(",", "").strip().rstrip(".")
    try:
        if "/" in s:
            a, b = s.split("/", 1)
            return float(a) / float(b)
        return float(s)
    except (ValueError, ZeroDivisionError):
        return None


def extract_answer(text: str) -> Optional[float]:
    for pat in _PATTERNS:
        m = pat.findall(text)
        if m:
            v = _to_float(m[-1])
            if v is not None:
                return v
    nums = _LAST.findall(text)
    return _to_float(nums[-1]) if nums else None


_STEPS = [re.compile(r"(步骤|step|第\s*\d+\s*步)", re.IGNORECASE), re.compile(r"\d+[.)]\s+\S")]


def check_format(text: str) -> bool:
    """True when the response shows its work or marks its answer: step markers ("Step 2", "1. ...", "第 3 步"),
    at least three lines, or an explicit answer marker (``####``, ``\\boxed{}``, "the answer is", "答案是")
    (src/reward/gsm8k_reward.py:74-99)."""
    if not text:
        return False
    has_steps = any(p.search(text) for p in _STEPS) or text.count("\n") >= 2
    return has_steps or any(p.search(text) for p in _PATTERNS)


def _same_number(pred: Optional[float], gt: Optional[float], tol: float) -> bool:
    """Equal answers: whole numbers must match exactly (9999 is not 10000, whatever the magnitude); otherwise within
    ``tol`` absolutely (1/3 against 0.3333) plus float noise.  The reference compares the normalised strings
    (src/reward/gsm8k_reward.py:102-125), which is exact for integers as well."""
    if pred is None or gt is None or pred != pred or gt != gt:
        return False
    if abs(pred) < 2 ** 53 and abs(gt) < 2 ** 53 and pred == int(pred) and gt == int(gt):
        return int(pred) == int(gt)
    return abs(pred - gt) <= max(tol, 1e-9 * abs(gt))


def compute_reward(response: str, ground_truth, tol: float = 1e-4) -> float:
    """+1.0 correct answer; otherwise -0.5 when the response is well formed (:func:`check_format`), -1.0 when it is
    not (src/reward/gsm8k_reward.py:102-125)."""
    pred = extract_answer(response or "")
    gt = ground_truth if isinstance(ground_truth, (int, float)) else extract_answer(str(ground_truth))
    if _same_number(pred, gt, tol):
        return 1.0
    return -0.5 if check_format(response or "") else -1.0


def compute_batch_rewards(responses: List[str], ground_truths: List) -> List[float]:
    assert len(responses) == len(ground_truths), \
        f"responses({len(responses)}) and ground_truths({len(ground_truths)}) must have same length"
    return [compute_reward(r, g) for r, g in zip(responses, ground_truths)]


class GSM8KRewardFunction:
    def __init__(self, correct: float = 1.0, wrong: float = -0.5, no_answer: float = -1.0, tol: float = 1e-4):
        self.correct, self.wrong, self.no_answer, self.tol = correct, wrong, no_answer, tol
        self.total = 0
        self.num_correct = 0
        self.num_formatted = 0
        self.reward_sum = 0.0

    def score(self, response: str, ground_truth) -> float:
        r = self._score(response, ground_truth)
        self.reward_sum += r
        return r

    def _score(self, response: str, ground_truth) -> float:
        self.total += 1
        formatted = check_format(response or "")
        self.num_formatted += int(formatted)
        pred = extract_answer(response or "")
        gt = ground_truth if isinstance(ground_truth, (int, float)) else extract_answer(str(ground_truth))
        if _same_number(pred, gt, self.tol):
            self.num_correct += 1
            return self.correct
        return self.wrong if formatted else self.no_answer

    def __call__(self, responses: List[List[str]], ground_truths: List) -> List[List[float]]:
        """``responses[b][k]`` -> rewards of the same shape."""
        return [[self.score(r, gt) for r in group] for group, gt in zip(responses, ground_truths)]

    @property
    def accuracy(self) -> float:
        return self.num_correct / self.total if self.total else 0.0

    @property
    def format_accuracy(self) -> float:
        """Share of scored responses that state their answer explicitly."""
        return self.num_formatted / self.total if self.total else 0.0

    @property
    def average_reward(self) -> float:
        return self.reward_sum / self.total if self.total else 0.0

    def get_stats(self) -> Dict[str, float]:
        return {"total": self.total, "accuracy": self.accuracy,
                "format_rate": self.num_formatted / self.total if self.total else 0.0}

    def reset_stats(self):
        self.total = self.num_correct = self.num_formatted = 0
        self.reward_sum = 0.0
