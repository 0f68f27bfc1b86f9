"""Text evaluation helpers: normalisation, token-F1, smoothed BLEU-4, exact match and an aggregate
(src/utils/eval_utils.py:22-178)."""
from __future__ import annotations

import math
import re
from collections import Counter
from dataclasses import dataclass, field
from typing import Dict, List


def normalize_text(s: str) -> str:
    """Lower-case, every character that is neither a word character, white space nor a CJK ideograph becomes a
    space (so ASCII and full-width punctuation both separate words), runs of white space collapse
    (src/utils/eval_utils.py:22-37)."""
    s = re.sub(r"[^\w\s\u4e00-\u9fff]", " ", s.lower())
    return " ".join(s.split())


def tokenize_for_eval(text: str) -> List[str]:
    """Evaluation tokens of mixed text: white-space words, except that a word containing CJK ideographs is split
    into its characters (src/utils/eval_utils.py:39-54)."""
    out: List[str] = []
    for word in normalize_text(text).split():
        if any("\u4e00" <= c <= "\u9fff" for c in word):
            out.extend(word)
        else:
            out.append(word)
    return out


def compute_exact_match(pred: str, ref: str) -> float:
    return float(normalize_text(pred) == normalize_text(ref))


def compute_token_f1(pred: str, ref: str) -> float:
    p, r = tokenize_for_eval(pred), tokenize_for_eval(ref)
    if not p or not r:
        return float(p == r)
    common = Counter(p) & Counter(r)
    n = sum(common.values())
    if n == 0:
        return 0.0
    prec, rec = n / len(p), n / len(r)
    return 2 * prec * rec / (prec + rec)


def compute_bleu4(pred: str, ref: str) -> float:
    """Sentence BLEU-4 with add-one smoothing on the higher-order precisions and brevity penalty."""
    p, r = tokenize_for_eval(pred), tokenize_for_eval(ref)
    if not p or not r:
        return 0.0
    logs = 0.0
    for n in range(1, 5):
        pn = Counter(tuple(p[i:i + n]) for i in range(len(p) - n + 1))
        rn = Counter(tuple(r[i:i + n]) for i in range(len(r) - n + 1))
        match = sum((pn & rn).values())
        total = max(sum(pn.values()), 0)
        if n == 1:
            if match == 0:
                return 0.0
            prec = match / total
        else:
            prec = (match + 1) / (total + 1)
        logs += 0.25 * math.log(prec)
    bp = 1.0 if len(p) > len(r) else math.exp(1 - len(r) / len(p))
    return bp * math.exp(logs)


@dataclass
class EvalMetrics:
    exact_match: List[float] = field(default_factory=list)
    f1: List[float] = field(default_factory=list)
    bleu4: List[float] = field(default_factory=list)

    def add(self, pred: str, ref: str):
        self.exact_match.append(compute_exact_match(pred, ref))
        self.f1.append(compute_token_f1(pred, ref))
        self.bleu4.append(compute_bleu4(pred, ref))

    def summary(self) -> Dict[str, float]:
        n = max(1, len(self.f1))
        return {"count": len(self.f1), "exact_match": sum(self.exact_match) / n, "token_f1": sum(self.f1) / n,
                "bleu4": sum(self.bleu4) / n}

    # ---- the reference's method names (src/utils/eval_utils.py:144-178) -----------------------------------------
    def compute_single(self, prediction: str, reference: str) -> Dict[str, float]:
        self.add(prediction, reference)
        return {"token_f1": self.f1[-1], "bleu4": self.bleu4[-1], "exact_match": self.exact_match[-1]}

    def compute_batch(self, predictions: List[str], references: List[str]) -> Dict[str, float]:
        """Scores every pair (they are kept for ``get_summary``) and returns this batch's averages."""
        assert len(predictions) == len(references) and predictions
        rows = [self.compute_single(p, r) for p, r in zip(predictions, references)]
        return {k: sum(r[k] for r in rows) / len(rows) for k in rows[0]}

    def get_summary(self) -> Dict[str, float]:
        """``<metric>_mean / _max / _min`` over everything scored so far (``{}`` when nothing was)."""
        out: Dict[str, float] = {}
        for k, v in (("token_f1", self.f1), ("bleu4", self.bleu4), ("exact_match", self.exact_match)):
            if v:
                out[f"{k}_mean"], out[f"{k}_max"], out[f"{k}_min"] = sum(v) / len(v), max(v), min(v)
        return out

    def reset(self):
        self.exact_match.clear()
        self.f1.clear()
        self.bleu4.clear()

