"""Data pipeline.

The reference imports ``src.data.data_pipeline`` (``GSM8KDataPipeline``, ``GRPOBatch``) but the file is
not part of its checkout; the contract below is the one its call sites use
(src/orchestrator/colocate_orchestrator.py:318-333,424,899,922-926): constructor keywords
``tokenizer_name, dataset_name, dataset_config, split, max_samples, prompt_template, prompt_field,
input_field, response_field, answer_field, dp_rank, dp_size``; attribute ``tokenizer``; ``len()``;
``get_batches(batch_size)`` yielding ``GRPOBatch(prompts, prompt_tokens, ground_truths,
reference_responses)``.  Samples are sharded by ``dp_rank / dp_size``.  Datasets and tokenizers are
loaded from local files only (no network): a JSON/JSONL file or a ``datasets`` directory on disk.
:class:`SyntheticTokenPipeline` provides the same interface over seeded random token ids.
"""
from __future__ import annotations

import json
import os
import random
from dataclasses import dataclass
from typing import Dict, Iterator, List, Optional

from ..obs.logging import get_logger

logger = get_logger("data.pipeline")

PROMPT_TEMPLATES: Dict[str, str] = {
    "qwen3_math": ("<|im_start|>system\nYou are a helpful math assistant. Solve the problem step by step and give "
                   "the final answer after '####'.<|im_end|>\n<|im_start|>user\n{prompt}<|im_end|>\n"
                   "<|im_start|>assistant\n"),
    "qwen3_instruction": ("<|im_start|>user\n{prompt}{input}<|im_end|>\n<|im_start|>assistant\n"),
    "plain": "{prompt}",
}


@dataclass
class GRPOBatch:
    prompts: List[str]
    prompt_tokens: List[List[int]]
    ground_truths: List
    reference_responses: Optional[List[str]] = None
    prompt_indices: Optional[List[int]] = None


class SimpleTokenizer:
    """Byte-level fallback tokenizer (ids 3..258; 0 pad, 1 bos, 2 eos) for runs without a HF tokenizer."""
    pad_token_id, bos_token_id, eos_token_id = 0, 1, 2
    vocab_size = 259

    def encode(self, text: str, add_special_tokens: bool = False) -> List[int]:
        ids = [b + 3 for b in text.encode("utf-8")]
        return ([self.bos_token_id] + ids) if add_special_tokens else ids

    def decode(self, ids, skip_special_tokens: bool = True) -> str:
        return bytes(i - 3 for i in ids if i >= 3 and i < 259).decode("utf-8", errors="replace")

    def __call__(self, text, **kw):
        return {"input_ids": self.encode(text)}


def _load_tokenizer(name: Optional[str]):
    if name and os.path.isdir(name):
        try:
            from transformers import AutoTokenizer
            return AutoTokenizer.from_pretrained(name, trust_remote_code=True, local_files_only=True)
        except Exception:  # noqa: BLE001 - fall back to bytes
            pass
    return SimpleTokenizer()


def _load_records(dataset_name: str, dataset_config: Optional[str], split: str) -> List[Dict]:
    if os.path.isfile(dataset_name):
        with open(dataset_name) as f:
            if dataset_name.endswith(".jsonl"):
                return [json.loads(l) for l in f if l.strip()]
            data = json.load(f)
            return data[split] if isinstance(data, dict) and split in data else data
    if os.path.isdir(dataset_name):
        plain = os.path.join(dataset_name, "data.jsonl")        # written by prepare_data.py without `datasets`
        if os.path.isfile(plain):
            with open(plain) as f:
                return [json.loads(l) for l in f if l.strip()]
        from datasets import load_from_disk
        ds = load_from_disk(dataset_name)
        ds = ds[split] if hasattr(ds, "keys") and split in ds else ds
        return [dict(r) for r in ds]
    raise FileNotFoundError(f"dataset {dataset_name!r} is not a local file or directory (no network access)")


class GSM8KDataPipeline:
    def __init__(self, tokenizer_name: Optional[str] = None, dataset_name: str = "gsm8k",
                 dataset_config: Optional[str] = "main", split: str = "train", max_samples: Optional[int] = None,
                 prompt_template: str = "qwen3_math", prompt_field: str = "question", input_field: str = "input",
                 response_field: str = "answer", answer_field: str = "answer", dp_rank: int = 0, dp_size: int = 1,
                 records: Optional[List[Dict]] = None, tokenizer=None, max_prompt_tokens: int = 1024):
        self.tokenizer = tokenizer if tokenizer is not None else _load_tokenizer(tokenizer_name)
        recs = records if records is not None else _load_records(dataset_name, dataset_config, split)
        if max_samples:
            recs = recs[:max_samples]
        # a record without a prompt would become an empty request; drop it here, before the shards are cut, so that
        # every rank drops the same ones
        usable = [r for r in recs if isinstance(r, dict) and str(r.get(prompt_field) if r.get(prompt_field) is not None
                                                                   else "").strip()]
        if len(usable) < len(recs):
            logger.warning("%d of %d records have no %r field (or an empty one) and are left out",
                           len(recs) - len(usable), len(recs), prompt_field)
        self.records = usable[dp_rank::max(1, dp_size)]
        self.template = PROMPT_TEMPLATES.get(prompt_template, prompt_template)
        self.prompt_field, self.input_field = prompt_field, input_field
        self.response_field, self.answer_field = response_field, answer_field
        self.dp_rank, self.dp_size, self.max_prompt_tokens = dp_rank, dp_size, max_prompt_tokens

    def __len__(self) -> int:
        return len(self.records)

    def format_prompt(self, rec: Dict) -> str:
        extra = rec.get(self.input_field) or ""
        return self.template.format(prompt=rec.get(self.prompt_field, ""), input=("\n" + extra) if extra else "")

    def get_batches(self, batch_size: int, shuffle: bool = False, seed: int = 0) -> Iterator[GRPOBatch]:
        order = list(range(len(self.records)))
        if shuffle:
            random.Random(seed).shuffle(order)
        for s in range(0, len(order) - batch_size + 1, batch_size):
            recs = [self.records[i] for i in order[s:s + batch_size]]
            prompts = [self.format_prompt(r) for r in recs]
            toks = [self.tokenizer.encode(p)[-self.max_prompt_tokens:] for p in prompts]
            yield GRPOBatch(prompts, toks, [r.get(self.answer_field) for r in recs],
                            [str(r.get(self.response_field, "")) for r in recs],
                            [order[s + j] * self.dp_size + self.dp_rank for j in range(len(recs))])


class SyntheticTokenPipeline:
    """Seeded uniform random prompts of a fixed length; ``prompts_share_prefix`` makes every group of
    ``group`` consecutive prompts share their first ``prefix_len`` tokens (prefix-cache workloads)."""

    def __init__(self, vocab_size: int, num_samples: int = 1024, prompt_len: int = 256, seed: int = 0,
                 dp_rank: int = 0, dp_size: int = 1, min_prompt_len: Optional[int] = None,
                 prefix_len: int = 0, group: int = 1, response_len: int = 0):
        self.tokenizer = SimpleTokenizer()
        self.vocab_size = vocab_size
        rng = random.Random(seed)
        self.samples: List[List[int]] = []
        self.responses: List[List[int]] = []
        prefix: List[int] = []
        for i in range(num_samples):
            if prefix_len and i % max(1, group) == 0:
                prefix = [rng.randrange(3, vocab_size) for _ in range(prefix_len)]
            n = prompt_len if min_prompt_len is None else rng.randint(min_prompt_len, prompt_len)
            body = [rng.randrange(3, vocab_size) for _ in range(max(0, n - len(prefix)))]
            self.samples.append((prefix + body)[:max(n, 1)])
            self.responses.append([rng.randrange(3, vocab_size) for _ in range(response_len)])
        self.index = list(range(dp_rank, num_samples, max(1, dp_size)))

    def __len__(self) -> int:
        return len(self.index)

    def get_batches(self, batch_size: int, shuffle: bool = False, seed: int = 0) -> Iterator[GRPOBatch]:
        order = list(self.index)
        if shuffle:
            random.Random(seed).shuffle(order)
        for s in range(0, len(order) - batch_size + 1, batch_size):
            idx = order[s:s + batch_size]
            yield GRPOBatch([f"<synthetic {i}>" for i in idx], [self.samples[i] for i in idx], idx,
                            None, idx)
