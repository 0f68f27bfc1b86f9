#!/usr/bin/env python
"""Prepare a local dataset file for the data pipeline: convert a Hugging Face dataset directory on disk
to JSONL, or synthesise an arithmetic GSM8K-style set when no dataset is available (no network)."""
import argparse
import json
import os
import random
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def synth(n, seed):
    rng = random.Random(seed)
    for _ in range(n):
        a, b, c = rng.randint(2, 99), rng.randint(2, 99), rng.randint(2, 9)
        yield {"question": f"Tom has {a} apples, buys {b} more and then splits them among {c} friends after giving away "
                           f"{(a + b) % c}. How many apples does each friend get?",
               "answer": f"He has {a}+{b}={a + b} apples. After giving away {(a + b) % c} he has {(a + b) - (a + b) % c}. "
                         f"Each friend gets {((a + b) - (a + b) % c) // c}. #### {((a + b) - (a + b) % c) // c}"}


def main():
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--source", default="", help="datasets directory saved with save_to_disk (optional)")
    ap.add_argument("--split", default="train")
    ap.add_argument("--out", default="data/gsm8k_train.jsonl")
    ap.add_argument("--num-synthetic", type=int, default=1000)
    ap.add_argument("--seed", type=int, default=0)
    a = ap.parse_args()
    os.makedirs(os.path.dirname(a.out) or ".", exist_ok=True)
    if a.source:
        from datasets import load_from_disk
        ds = load_from_disk(a.source)
        ds = ds[a.split] if hasattr(ds, "keys") and a.split in ds else ds
        rows = (dict(r) for r in ds)
    else:
        rows = synth(a.num_synthetic, a.seed)
    n = 0
    with open(a.out, "w") as f:
        for r in rows:
            f.write(json.dumps(r) + "\n")
            n += 1
    print(f"wrote {n} records to {a.out}")


if __name__ == "__main__":
    main()
