#!/usr/bin/env python
"""Runs the benchmark matrix (SFT throughput per ZeRO stage, inference variants, GRPO iteration, weight
sync) as child processes and collects their JSON lines into one report.

    python scripts/benchmark_all.py --gpus 8 --out outputs/benchmark_all.json
"""
import argparse
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run(cmd, timeout):
    print("+", " ".join(cmd), file=sys.stderr)
    try:
        r = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, cwd=ROOT)
    except subprocess.TimeoutExpired:
        return {"error": "timeout", "cmd": cmd}
    for line in reversed(r.stdout.strip().splitlines()):
        line = line.strip()
        if line.startswith("{"):
            try:
                return json.loads(line)
            except json.JSONDecodeError:
                continue
    return {"error": f"rc={r.returncode}", "stderr": r.stderr[-2000:], "cmd": cmd}


def torchrun(n, script, *args):
    if n == 1:
        return [sys.executable, script, *args]
    return [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
            "--master-addr", "127.0.0.1", "--master-port", "29533", script, *args]


def main():
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=6)
    ap.add_argument("--out", default="outputs/benchmark_all.json")
    ap.add_argument("--skip-reference", action="store_true")
    ap.add_argument("--timeout", type=int, default=1800)
    a = ap.parse_args()
    rep = {"sft": {}, "inference": {}, "rl": {}}
    for stage in (1, 2, 3):
        rep["sft"][f"zero{stage}"] = run(torchrun(a.gpus, "bench.py", "--gpus", str(a.gpus), "--steps", str(a.steps),
                                                  "--warmup", "3", "--zero-stage", str(stage)), a.timeout)
    if not a.skip_reference:
        rep["sft"]["reference_zero1"] = run(torchrun(a.gpus, "bench.py", "--impl", "reference", "--gpus", str(a.gpus),
                                                     "--steps", str(a.steps), "--warmup", "3"), a.timeout)
    inf = "scripts/benchmark_inference.py"
    rep["inference"]["fp16"] = run([sys.executable, inf], a.timeout)
    rep["inference"]["fp8"] = run([sys.executable, inf, "--kv-cache-dtype", "fp8"], a.timeout)
    rep["inference"]["cuda_graph"] = run([sys.executable, inf, "--cuda-graph"], a.timeout)
    rep["inference"]["speculative"] = run([sys.executable, inf, "--speculative", "--num-requests", "8"], a.timeout)
    rep["inference"]["long_32k"] = run([sys.executable, inf, "--long-context", "32768", "--output-tokens", "64"], a.timeout)
    rep["rl"]["grpo_colocate"] = run(torchrun(a.gpus, "scripts/benchmark_grpo.py", "--iterations", "3"), a.timeout)
    os.makedirs(os.path.dirname(os.path.join(ROOT, a.out)), exist_ok=True)
    with open(os.path.join(ROOT, a.out), "w") as f:
        json.dump(rep, f, indent=2)
    print(json.dumps(rep, indent=2))


if __name__ == "__main__":
    main()
