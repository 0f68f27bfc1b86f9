"""Entry-point scripts: the reference's command-line flags are accepted, and the small flows run on CPU."""
import importlib.util
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# flags of the reference's scripts (scripts/*.py of the reference project) that a user may have in a launcher
REFERENCE_FLAGS = {
    "run_inference.py": ["--model", "-m", "--mode", "--prompt", "-p", "--input", "-i", "--output", "-o", "--max-tokens",
                         "--temperature", "--top-p", "--batch-size", "--num-samples", "--interactive", "--config",
                         "--num-blocks", "--block-size", "--enable-prefix-cache", "--enable-cuda-graph", "--enable-async",
                         "--enable-partitioned-attn"],
    "run_colocate.py": ["--config", "--model", "--tp-size", "--dp-size", "--iterations", "--batch-size", "--num-samples",
                        "--training-mode", "--inference-backend", "--vllm-url", "--lr", "--lora-rank", "--max-tokens",
                        "--resume-from", "--log-file"],
    "run_disaggregated.py": ["--model", "--train-tp", "--infer-tp", "--iterations", "--batch-size", "--num-samples",
                             "--weight-backend", "--no-overlap", "--lr", "--lora-rank", "--max-tokens", "--log-file"],
    "benchmark_all.py": ["--model", "--iterations", "--batch-size", "--num-samples", "--quick", "--vllm-url", "--output",
                         "--tp-size", "--train-tp", "--infer-tp"],
    "prepare_data.py": ["--dataset", "--config", "--split", "--output", "--max-samples", "--required-field"],
    "profile_memory.py": ["--config", "--output", "--device", "--skip-backward"],
}


def _load(name):
    spec = importlib.util.spec_from_file_location(name[:-3], os.path.join(ROOT, "scripts", name))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


@pytest.mark.parametrize("script", sorted(REFERENCE_FLAGS))
def test_reference_flags_are_accepted(script):
    r = subprocess.run([sys.executable, os.path.join(ROOT, "scripts", script), "--help"], capture_output=True, text=True,
                       timeout=300)
    assert r.returncode == 0, r.stderr[-500:]
    words = set(r.stdout.replace(",", " ").replace("[", " ").replace("]", " ").split())
    missing = [f for f in REFERENCE_FLAGS[script] if f not in words]
    assert not missing, f"{script}: flags of the reference not accepted: {missing}"


def test_run_inference_jsonl_in_jsonl_out(tmp_path, capsys):
    src = tmp_path / "prompts.jsonl"
    src.write_text('"hello there"\n{"prompt": "two plus two"}\n\n{"text": "third"}\n')
    out = tmp_path / "out.jsonl"
    mod = _load("run_inference.py")
    assert mod.load_prompts_from_file(str(src)) == ["hello there", "two plus two", "third"]
    mod.main(["--model-preset", "tiny128", "--mode", "kv_cache", "-i", str(src), "-p", "from the cli", "--num-samples", "2",
              "--batch-size", "3", "--max-tokens", "4", "-o", str(out), "--enable-prefix-cache", "--num-blocks", "64"])
    rows = [json.loads(l) for l in out.read_text().splitlines()]
    assert len(rows) == 8 and [r["sample_idx"] for r in rows[:2]] == [0, 1]
    assert rows[0]["prompt"] == "from the cli" and rows[-1]["prompt"] == "third"
    assert all(0 < r["num_tokens"] <= 4 and set(r) == {"prompt", "sample_idx", "output", "num_tokens", "time_s",
                                                       "tokens_per_s"} for r in rows)
    summary = json.loads(capsys.readouterr().out)
    assert summary["prompts"] == 4 and summary["samples"] == 8 and summary["mode"] == "kv_cache"


def test_run_inference_reads_both_yaml_dialects(tmp_path):
    mod = _load("run_inference.py")
    ref = tmp_path / "ref.yaml"
    ref.write_text("model:\n  path: ''\ninference:\n  mode: mock\n  max_tokens: 5\n  temperature: 0.3\n  top_p: 0.5\n"
                   "kv_cache:\n  num_blocks: 48\n  block_size: 16\n  enable_prefix_caching: true\n  enable_cuda_graph: true\n"
                   "advanced:\n  enable_partitioned_attention: true\n  use_radix_cache: true\n  enable_async_scheduling: true\n")
    from b200fw.config import load_yaml_config
    a = mod.parse_args(["--config", str(ref), "--model-preset", "tiny128"])
    c = mod.create_inference_config(a, load_yaml_config(str(ref)))
    assert (c.inference_mode, c.temperature, c.top_p, c.num_blocks) == ("mock", 0.3, 0.5, 48)
    assert c.enable_prefix_caching and c.enable_cuda_graph and c.enable_partitioned_attention and c.use_radix_cache
    assert c.enable_async_scheduling
    own = os.path.join(ROOT, "configs", "inference", "standalone.yaml")
    a = mod.parse_args(["--config", own, "--temperature", "0.1", "--num-blocks", "32"])       # the command line wins
    c = mod.create_inference_config(a, load_yaml_config(own))
    assert c.temperature == 0.1 and c.num_blocks == 32 and c.top_p == 0.95 and c.use_radix_cache and c.chunk_size == 512


def test_run_inference_interactive_reads_until_quit():
    import io
    mod = _load("run_inference.py")
    a = mod.parse_args(["--model-preset", "tiny128", "--mode", "mock", "--interactive", "--max-tokens", "3"])
    cfg = mod.create_inference_config(a, {})
    eng = mod.InferenceEngine(cfg).initialize()
    from b200fw.data import SimpleTokenizer
    lines = []
    mod.run_interactive(eng, SimpleTokenizer(), a, 3, cfg.vocab_size, stdin=io.StringIO("first\n\nsecond\nquit\nnever\n"),
                        out=lines.append)
    assert len(lines) == 3 and lines[1].startswith("[") and "tok/s" in lines[2]


def test_prepare_data_file_directory_and_required_fields(tmp_path):
    mod = _load("prepare_data.py")
    f = tmp_path / "syn.jsonl"
    assert mod.main(["--dataset", "synthetic", "--num-synthetic", "30", "--max-samples", "12", "--output", str(f),
                     "--required-field", "question", "--required-field", "answer"]) == 0
    rows = [json.loads(l) for l in f.read_text().splitlines()]
    assert len(rows) == 12 and "####" in rows[0]["answer"]
    man = json.load(open(str(f) + ".manifest.json"))
    assert man["rows"] == 12 and man["required_fields"] == ["question", "answer"] and man["split"] == "train"
    with pytest.raises(ValueError, match="missing required field"):
        mod.main(["--dataset", str(f), "--output", str(tmp_path / "x.jsonl"), "--required-field", "nope"])
    d = tmp_path / "as_dir"
    assert mod.main(["--dataset", str(f), "--output", str(d), "--max-samples", "5"]) == 0
    assert json.load(open(d / "train_infer_manifest.json"))["rows"] == 5
    from b200fw.data.pipeline import GSM8KDataPipeline
    assert len(GSM8KDataPipeline(None, str(d))) == 5          # the pipeline reads what the script wrote
    from b200fw.reward import GSM8KRewardFunction
    assert GSM8KRewardFunction().score(rows[0]["answer"], rows[0]["answer"]) == 1.0


def test_profile_memory_from_yaml(tmp_path):
    mod = _load("profile_memory.py")
    out = tmp_path / "rep" / "memory_report.json"
    rep = mod.main(["--config", os.path.join(ROOT, "configs", "training", "sft.yaml"), "--model-preset", "tiny128",
                    "--batch-size", "2", "--seq-len", "64", "--device", "cpu", "--skip-backward", "--output", str(out)])
    d = json.load(open(out))
    assert set(d) >= {"breakdown", "phase_peaks", "optimizer_bytes"} and "forward" in d["phase_peaks"] and rep is not None


def test_sigterm_stops_run_colocate_at_an_iteration_boundary_and_the_checkpoint_resumes(tmp_path):
    """The whole path a preempted job takes: ``run_colocate.py`` gets SIGTERM while it trains, finishes the iteration,
    writes ``iter_N`` / ``latest`` with the orchestrator's position and exits 0; a second launch with ``--resume-from``
    continues at iteration N."""
    import signal
    import time
    cfg = tmp_path / "cfg.yaml"
    cfg.write_text(f"""
model: {{preset: tiny128, max_seq_len: 64}}
runtime: {{precision: fp32, inference_backend: native}}
training: {{mode: sft, total_iterations: 1000000, batch_size: 2, gradient_accumulation_steps: 1, warmup_steps: 0}}
lora: {{rank: 0}}
checkpoint: {{save_dir: {tmp_path}/ckpt}}
experiment: {{output_dir: {tmp_path}/out}}
inference_preview: {{enabled: false, max_tokens: 4}}
""")
    cmd = [sys.executable, os.path.join(ROOT, "scripts", "run_colocate.py"), "--config", str(cfg), "--synthetic"]
    p = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    try:
        metrics = tmp_path / "out" / "metrics_rank0.jsonl"
        deadline = time.time() + 240
        while time.time() < deadline and not (metrics.exists() and metrics.stat().st_size > 0):
            assert p.poll() is None, p.stdout.read()
            time.sleep(0.2)
        assert metrics.exists(), "the run never recorded an iteration"
        p.send_signal(signal.SIGTERM)            # the exact child started above
        out, _ = p.communicate(timeout=120)
    finally:
        if p.poll() is None:
            p.kill()
    assert p.returncode == 0, out[-2000:]
    assert "stopping after the current iteration" in out
    state = json.load(open(tmp_path / "ckpt" / "latest" / "orchestrator_state.json"))
    done = state["iterations_completed"]
    assert done >= 1 and os.path.isdir(tmp_path / "ckpt" / f"iter_{done}") and not os.path.exists(tmp_path / "ckpt" / "final")
    cfg.write_text(cfg.read_text().replace("total_iterations: 1000000", f"total_iterations: {done + 2}"))
    r = subprocess.run(cmd + ["--resume-from", str(tmp_path / "ckpt" / "latest")], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, (r.stdout + r.stderr)[-2000:]
    assert f"continuing at iteration {done} of {done + 2}" in r.stdout + r.stderr
    assert json.loads(r.stdout[r.stdout.index("{"):])["completed_iterations"] == 2
