#!/usr/bin/env python
"""Prepare a local dataset for the data pipeline (flags after the reference's scripts/prepare_data.py:16-30):

    python scripts/prepare_data.py --dataset gsm8k --config main --split train --output data/gsm8k --required-field question
    python scripts/prepare_data.py --dataset synthetic --num-synthetic 2000 --output data/gsm8k_train.jsonl

Reads a hub dataset (when there is network access), a ``save_to_disk`` directory or a JSON / JSONL file, or
synthesises an arithmetic GSM8K-style set; writes a JSONL file or a ``save_to_disk`` directory plus a manifest."""
import argparse
import json
import os
import random
import sys
from datetime import datetime, timezone

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def synth(n, seed):
    rng = random.Random(seed)
    for _ in range(n):
        a, b, c = rng.randint(2, 99), rng.randint(2, 99), rng.randint(2, 9)
        yield {"question": f"Tom has {a} apples, buys {b} more and then splits them among {c} friends after giving away "
                           f"{(a + b) % c}. How many apples does each friend get?",
               "answer": f"He has {a}+{b}={a + b} apples. After giving away {(a + b) % c} he has {(a + b) - (a + b) % c}. "
                         f"Each friend gets {((a + b) - (a + b) % c) // c}. #### {((a + b) - (a + b) % c) // c}"}


def load_rows(a):
    """Rows from, in order: ``--dataset synthetic`` (or nothing given), a local JSON / JSONL file, a directory
    written by ``save_to_disk``, a Hugging Face hub name (needs network access and the ``datasets`` package)."""
    src = a.dataset or a.source
    if not src or src == "synthetic":
        return list(synth(a.num_synthetic, a.seed))
    if os.path.isfile(src):
        with open(src) as f:
            if src.endswith(".jsonl"):
                return [json.loads(line) for line in f if line.strip()]
            data = json.load(f)
            return data[a.split] if isinstance(data, dict) and a.split in data else data
    if os.path.isdir(src):
        from datasets import load_from_disk
        ds = load_from_disk(src)
        ds = ds[a.split] if hasattr(ds, "keys") and a.split in ds else ds
        return [dict(r) for r in ds]
    from datasets import load_dataset
    ds = load_dataset(src, a.config, split=a.split) if a.config else load_dataset(src, split=a.split)
    return [dict(r) for r in ds]


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--dataset", default="", help="'synthetic', a local .json/.jsonl file, a save_to_disk directory, "
                                                  "or a Hugging Face dataset name")
    ap.add_argument("--config", default=None, help="dataset config name (hub datasets)")
    ap.add_argument("--split", default="train")
    ap.add_argument("--output", "--out", dest="output", default="data/gsm8k_train.jsonl",
                    help="a .jsonl file, or a directory (written with save_to_disk when `datasets` is installed)")
    ap.add_argument("--max-samples", type=int, default=None)
    ap.add_argument("--required-field", action="append", default=[],
                    help="field every row must have (checked on the first 20 rows); repeatable")
    ap.add_argument("--source", default="", help="older name of --dataset for a save_to_disk directory")
    ap.add_argument("--num-synthetic", type=int, default=1000)
    ap.add_argument("--seed", type=int, default=0)
    a = ap.parse_args(argv)
    rows = load_rows(a)
    if a.max_samples is not None:
        rows = rows[:a.max_samples]
    missing = sorted({f for f in a.required_field for r in rows[:20] if f not in r})
    if missing:
        raise ValueError(f"Dataset is missing required field(s): {', '.join(missing)}")
    out = os.path.abspath(a.output)
    as_file = out.endswith(".jsonl") or out.endswith(".json")
    os.makedirs(os.path.dirname(out) if as_file else out, exist_ok=True)
    if as_file:
        with open(out, "w") as f:
            for r in rows:
                f.write(json.dumps(r, ensure_ascii=False) + "\n")
        manifest_path = out + ".manifest.json"
    else:
        try:
            from datasets import Dataset
            Dataset.from_list(rows).save_to_disk(out)
        except ImportError:
            with open(os.path.join(out, "data.jsonl"), "w") as f:
                for r in rows:
                    f.write(json.dumps(r, ensure_ascii=False) + "\n")
        manifest_path = os.path.join(out, "train_infer_manifest.json")
    manifest = {"dataset": a.dataset or a.source or "synthetic", "config": a.config, "split": a.split, "rows": len(rows),
                "output": out, "required_fields": a.required_field,
                "created_at": datetime.now(timezone.utc).isoformat()}
    with open(manifest_path, "w", encoding="utf-8") as f:
        json.dump(manifest, f, ensure_ascii=False, indent=2)
    print(json.dumps(manifest, ensure_ascii=False, indent=2))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
