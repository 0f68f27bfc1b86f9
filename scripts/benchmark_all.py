#!/usr/bin/env python
"""Runs the benchmark matrix (SFT throughput per ZeRO stage, inference variants, GRPO iteration, weight
sync) as child processes and collects their JSON lines into one report.

    python scripts/benchmark_all.py --gpus 8 --output outputs/benchmark_all.json
    python scripts/benchmark_all.py --gpus 4 --quick --iterations 3 --batch-size 16 --num-samples 4

The ``architectures`` section compares colocate with disaggregated GRPO on one workload (the reference's
benchmark_all.py does only this); ``--train-tp`` / ``--infer-tp`` size the two rank groups.
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
    start = r.stdout.find("{")                    # a pretty-printed (multi-line) JSON document
    if start >= 0:
        try:
            return json.loads(r.stdout[start:])
        except json.JSONDecodeError:
            pass
    return {"error": f"rc={r.returncode}", "stderr": r.stderr[-2000:], "cmd": cmd}


def torchrun(n, script, *args):
    if n == 1:
        return [sys.executable, script, *args]
    return [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
            "--master-addr", "127.0.0.1", "--master-port", "29533", script, *args]


def architectures(a):
    """Colocate against disaggregated GRPO on the same workload (what the reference's benchmark_all.py measures:
    scripts/benchmark_all.py:60-160), as child processes under torchrun."""
    model = ["--model-preset", a.model_preset] if not a.model else []
    out = {}
    out["colocate"] = run(torchrun(a.gpus, "scripts/benchmark_grpo.py", *model, "--iterations", str(a.iterations),
                                   "--prompts", str(a.batch_size), "--num-samples", str(a.num_samples)), a.timeout)
    if a.quick:
        out["disaggregated"] = {"status": "skipped", "reason": "--quick"}
    elif a.train_tp + a.infer_tp > max(a.gpus, 2):
        out["disaggregated"] = {"status": "skipped", "reason": f"needs {a.train_tp + a.infer_tp} GPUs"}
    else:
        margs = ["--model", a.model] if a.model else model
        out["disaggregated"] = run(torchrun(a.train_tp + a.infer_tp, "scripts/run_disaggregated.py", *margs,
                                            "--train-tp", str(a.train_tp), "--infer-tp", str(a.infer_tp),
                                            "--iterations", str(a.iterations), "--batch-size", str(a.batch_size),
                                            "--num-samples", str(a.num_samples)), a.timeout)
    return out


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=6)
    ap.add_argument("--output", "--out", dest="out", default=None, help="report path (default: outputs/benchmark_TIMESTAMP.json)")
    ap.add_argument("--skip-reference", action="store_true")
    ap.add_argument("--timeout", type=int, default=1800)
    # the reference's flags (colocate against disaggregated)
    ap.add_argument("--model", default="", help="HF model directory (default: the --model-preset architecture, random init)")
    ap.add_argument("--model-preset", default="qwen3-0.6b")
    ap.add_argument("--iterations", type=int, default=3)
    ap.add_argument("--batch-size", type=int, default=64, help="prompts per GRPO iteration")
    ap.add_argument("--num-samples", type=int, default=8, help="responses per prompt")
    ap.add_argument("--quick", action="store_true", help="skip the disaggregated run and the SFT / inference matrix")
    ap.add_argument("--vllm-url", default="http://localhost:8000", help="accepted for compatibility; rollouts use the native engine")
    ap.add_argument("--tp-size", type=int, default=1, help="accepted for compatibility (colocate rollouts need tp 1)")
    ap.add_argument("--train-tp", type=int, default=2, help="trainer ranks of the disaggregated run")
    ap.add_argument("--infer-tp", type=int, default=2, help="rollout ranks of the disaggregated run")
    a = ap.parse_args(argv)
    if a.out is None:
        import time
        a.out = os.path.join("outputs", f"benchmark_{time.strftime('%Y%m%d_%H%M%S')}.json")
    rep = {"sft": {}, "inference": {}, "rl": {}, "architectures": architectures(a)}
    if not a.quick:
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
    rep["rl"]["grpo_colocate"] = rep["architectures"]["colocate"]
    path = a.out if os.path.isabs(a.out) else os.path.join(ROOT, a.out)
    os.makedirs(os.path.dirname(path), exist_ok=True)
    with open(path, "w") as f:
        json.dump(rep, f, indent=2)
    print(json.dumps(rep, indent=2))
    return rep


if __name__ == "__main__":
    main()
