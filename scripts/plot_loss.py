#!/usr/bin/env python
"""Print (and optionally save as CSV) a scalar series from a run's TensorBoard event files.

    python scripts/plot_loss.py outputs/sft/qwen3_0_6b/tensorboard            # train/loss
    python scripts/plot_loss.py outputs/run/tensorboard --tag train/lr --csv lr.csv

Reads the event files directly, so the ``tensorboard`` package is not needed
(the reference's helper: _plot_loss.py:1-20).
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from b200fw.obs.tb_events import read_scalars  # noqa: E402


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("logdir", nargs="?", default="outputs/sft/qwen3_0_6b/tensorboard")
    ap.add_argument("--tag", default="train/loss")
    ap.add_argument("--csv", default=None, help="also write step,value rows to this file")
    a = ap.parse_args(argv)
    if not os.path.exists(a.logdir):
        print(f"no such log directory: {a.logdir}")
        return 1
    scalars = read_scalars(a.logdir)
    print(f"Available tags: {sorted(scalars)}\n")
    series = scalars.get(a.tag)
    if not series:
        print(f"No {a.tag} found")
        return 1
    print("     Step |    Value")
    print("----------|----------")
    for step, value, _ in series:
        print(f"  {step:>7} | {value:.4f}")
    if a.csv:
        with open(a.csv, "w") as f:
            f.write("step,value\n")
            for step, value, _ in series:
                f.write(f"{step},{value}\n")
    return 0


if __name__ == "__main__":
    sys.exit(main())
