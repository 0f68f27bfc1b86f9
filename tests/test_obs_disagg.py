"""Observability helpers (metrics, event files, NVTX, profilers, timeline, memory, eval) and the disaggregated loop over gloo."""
import json
import os
import tempfile

from b200fw.obs import (ArtifactWriter, CommProfiler, ComputeProfiler, EvalMetrics, MemoryBreakdown, MemoryManager,
                        MemoryProfiler, MemoryReport, MetricsCollector, ScheduleVisualizer, compute_bleu4,
                        compute_exact_match, compute_token_f1, get_logger, setup_logger)


def test_event_files_round_trip_without_the_tensorboard_package(capsys):
    """Scalar event files: CRC-32C check value, TFRecord framing, proto fields, the loss-printing helper."""
    import importlib.util
    from b200fw.obs.tb_events import EventFileWriter, crc32c, read_scalars
    assert crc32c(b"123456789") == 0xE3069283                      # the standard CRC-32C check value
    with tempfile.TemporaryDirectory() as d:
        with EventFileWriter(d) as w:
            for i in range(4):
                w.add_scalar("train/loss", 2.0 - 0.25 * i, i)
            w.add_scalar("train/lr", 1e-5, 300)
        m = MetricsCollector()
        m.record("reward", 0.5, 7)
        with EventFileWriter(d) as w2:
            m.export_tensorboard(w2, "rollout/")
        files = [f for f in os.listdir(d) if "tfevents" in f]
        assert files and all(f.startswith("events.out.tfevents.") for f in files)
        sc = read_scalars(d)
        assert [(s, v) for s, v, _ in sc["train/loss"]] == [(0, 2.0), (1, 1.75), (2, 1.5), (3, 1.25)]
        assert sc["train/lr"][0][0] == 300 and abs(sc["train/lr"][0][1] - 1e-5) < 1e-12
        assert sc["rollout/reward"][0][:2] == (7, 0.5)
        # a flipped payload byte is caught by the record checksum
        path = os.path.join(d, sorted(files)[0])
        raw = bytearray(open(path, "rb").read())
        raw[-6] ^= 0xFF
        bad = os.path.join(d, "bad.tfevents")
        open(bad, "wb").write(bytes(raw))
        try:
            read_scalars(bad)
            raise AssertionError("corruption not detected")
        except ValueError:
            pass
        os.remove(bad)
        spec = importlib.util.spec_from_file_location(
            "plot_loss", os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "scripts", "plot_loss.py"))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        assert mod.main([d]) == 0
        out = capsys.readouterr().out
        assert "train/loss" in out and "1.7500" in out
        assert mod.main([d, "--tag", "missing"]) == 1


def test_nvtx_ranges_are_free_when_off_and_balanced_when_on():
    from b200fw.obs import nvtx
    was = nvtx.enabled()
    try:
        nvtx.enable(False)
        assert nvtx.range("a") is nvtx.range("b")               # shared no-op context
        calls = []

        @nvtx.annotate("unit/fn")
        def f(x):
            calls.append(x)
            return x + 1

        assert f(1) == 2
        before = nvtx._state["pushed"]
        nvtx.enable(True)
        with nvtx.range("outer"):
            with nvtx.range("inner"):
                assert f(2) == 3
        assert nvtx._state["pushed"] == before + 3 and calls == [1, 2]
    finally:
        nvtx.enable(was)


def test_metrics_collector_and_artifacts():
    m = MetricsCollector()
    for i, v in enumerate([1.0, 2.0, 3.0]):
        m.record("loss", v, i)
    with m.timer("step"):
        pass
    s = m.summary()
    assert s["loss"]["mean"] == 2.0 and s["loss"]["last"] == 3.0 and s["step"]["count"] == 1
    assert m.get_latest("loss") == 3.0 and m.get_average("loss", last_n=2) == 2.5

    class TB:
        def __init__(self):
            self.rows = []

        def add_scalar(self, k, v, s):
            self.rows.append((k, v, s))

    tb = TB()
    m.export_tensorboard(tb, "train/")
    assert tb.rows[0] == ("train/loss", 1.0, 0)
    with tempfile.TemporaryDirectory() as d:
        w0, w1 = ArtifactWriter(d, 0, 2), ArtifactWriter(d, 1, 2)
        assert w0.write_json("run_summary.json", {"a": 1}) and w1.write_json("run_summary.json", {"a": 2}) is None
        w1.append_jsonl("metrics", {"x": 1})
        w1.write_json("memory_timeline.json", [1], all_ranks=True)
        assert sorted(os.listdir(d)) == ["memory_timeline_rank1.json", "metrics_rank1.jsonl", "run_summary.json"]
        assert json.load(open(os.path.join(d, "run_summary.json"))) == {"a": 1}


def test_profilers_formulas():
    assert abs(CommProfiler.bus_bandwidth("all_reduce", 10 ** 9, 8, 1.0) - 1750.0) < 1e-6
    assert abs(CommProfiler.bus_bandwidth("all_gather", 8 * 10 ** 8, 8, 1.0) - 700.0) < 1e-6
    r = CommProfiler.fused_roofline(flops=1.0737e12, wire_bytes=146.8e6, ms=1.2, peak_tflops=1392.7, link_gbs=770.0)
    assert r["bound"] == "compute" and abs(r["t_compute_ms"] - 0.771) < 0.01 and 0.6 < r["fraction"] < 0.7
    cp = CommProfiler()
    cp.add("all_reduce", 1 << 20, 8, 0.1)
    cp.set_step_time(1.0)
    s = cp.get_summary()
    assert s["ops"]["all_reduce"]["count"] == 1 and abs(s["comm_ratio"] - 0.1) < 1e-9
    # the reference formula: L*2*B*S*(4H^2+3HI) + 2*B*S*H*V, x3 for full fine-tuning
    f = ComputeProfiler.reference_formula_flops(L=2, B=1, S=4, H=8, I=16, V=32, full=True)
    assert f == 3 * (2 * 2 * 4 * (4 * 64 + 3 * 8 * 16) + 2 * 4 * 8 * 32)
    from b200fw.model import PRESETS
    ex = ComputeProfiler.exact_flops(PRESETS["qwen3-0.6b"], 8, 1024)
    assert 3.0e13 < ex < 3.4e13
    prof = ComputeProfiler(peak_tflops=1000.0)
    assert abs(prof.compute_mfu(5e14, 1.0) - 0.5) < 1e-9


def test_timeline_gantt_and_chrome_trace():
    v = ScheduleVisualizer()
    v.add_event("F0", "forward", "stage0", 0, 10)
    v.add_event("B0", "backward", "stage0", 20, 40)
    v.add_event("F0", "forward", "stage1", 10, 20)
    g = v.ascii_gantt(40)
    assert "stage0" in g and "F" in g and "B" in g
    tr = v.chrome_trace()
    assert len([e for e in tr["traceEvents"] if e["ph"] == "X"]) == 3
    u = v.utilisation()
    assert abs(u["stage0"]["utilisation"] - 0.75) < 1e-9 and abs(u["stage1"]["bubble_ratio"] - 0.75) < 1e-9
    assert ScheduleVisualizer.compare(v, v)["speedup"] == 1.0


def test_memory_helpers_on_cpu():
    p = MemoryProfiler()
    s = p.snapshot("x")
    assert s.allocated_gb == 0.0 and p.timeline()[0]["tag"] == "x"
    b = MemoryBreakdown.estimate(600_000_000, dp=8, zero_stage=3, batch_tokens=8192, hidden=1024, layers=28,
                                 vocab=151936, intermediate=3072)
    b1 = MemoryBreakdown.estimate(600_000_000, dp=8, zero_stage=1, batch_tokens=8192, hidden=1024, layers=28,
                                  vocab=151936, intermediate=3072)
    assert b.params_gb < b1.params_gb and b.grads_gb < b1.grads_gb and abs(b.optimizer_gb - b1.optimizer_gb) < 1e-9
    rep = MemoryReport.from_profiler(p, b)
    assert "static estimate" in rep.to_text() and rep.to_dict()["breakdown"]["total_gb"] > 0
    assert MemoryManager().check() == "ok"


def test_eval_utils_and_logger(tmp_path):
    assert compute_exact_match("The  Answer.", "the answer") == 1.0 and compute_exact_match("The Answer.", "answer") == 0.0
    assert abs(compute_token_f1("cat sat", "cat sat down") - 0.8) < 1e-9
    from b200fw.obs.eval_utils import normalize_text, tokenize_for_eval
    assert normalize_text("Hello, World!  x=3") == "hello world x 3" and normalize_text("答案是：18。") == "答案是 18"
    assert tokenize_for_eval("The answer 是18个苹果, ok") == ["the", "answer", "是", "1", "8", "个", "苹", "果", "ok"]
    assert abs(compute_token_f1("答案是十八", "答案是十九") - 0.8) < 1e-9
    assert compute_bleu4("the quick brown fox jumps", "the quick brown fox jumps") == 1.0
    assert 0 < compute_bleu4("the quick brown dog jumps high", "the quick brown fox jumps high") < 1
    e = EvalMetrics()
    e.add("42", "42")
    e.add("x", "y")
    assert e.summary()["exact_match"] == 0.5
    log = tmp_path / "run.log"
    setup_logger(log_file=str(log))
    get_logger("test").info("hello %d", 7)
    assert "[INFO] [b200fw.test] hello 7" in log.read_text()
    setup_logger()


def _disagg_worker(rank, world, mode):
    import torch.distributed as dist
    from b200fw.dist.context import ParallelContext
    from b200fw.infer import InferenceConfig, InferenceEngine
    from b200fw.model import PRESETS, ModelConfig, ParallelTransformerModel
    from b200fw.orch import DisaggConfig, DisaggOrchestrator
    from b200fw.train import TrainConfig, TrainEngine
    dist.init_process_group("gloo", rank=rank, world_size=world)
    mode_arg = mode
    use_data = mode.endswith("+data")
    mode = mode.split("+")[0]
    mc = ModelConfig(vocab_size=320 if use_data else 128, hidden_size=32, num_layers=2, num_heads=2, num_kv_heads=2, head_dim=16,
                     intermediate_size=48, max_position_embeddings=128, tie_word_embeddings=True)
    cfg = DisaggConfig(num_train_gpus=2, num_infer_gpus=2, total_iterations=2, batch_size=4, num_samples_per_prompt=2,
                       prompt_len=8, max_tokens=5, mode=mode, kv_num_blocks=64,
                       # without CUDA peer memory the peer-write request falls back to the collective broadcast
                       transfer_backend="peer_write" if mode == "sequential" else "nccl",
                       heartbeat_interval_s=0.05 if mode_arg.endswith("+leave") else 0.0, heartbeat_timeout_s=2.0)

    def trainer(group, n, r):
        ctx = ParallelContext(1, n, 1, r, n, r, "gloo")
        ctx.dp_group, ctx.dp_ranks = group, list(range(n))
        ParallelContext._instance = ctx
        tc = TrainConfig(model_config=mc, dp_size=n, lora_rank=0, zero_stage=2, gradient_accumulation_steps=1,
                         grpo_beta=0.0, max_seq_len=32, warmup_steps=0, use_amp=False, amp_dtype="fp32", learning_rate=1e-3)
        return TrainEngine(tc).initialize(ctx)

    def engine(i):
        m = ParallelTransformerModel(mc)
        m.init_weights(0)
        ic = InferenceConfig.from_model_config(mc, num_blocks=64, inference_mode="kv_cache", seed=i, eos_token_id=None)
        return InferenceEngine(ic, m).initialize()

    data = None
    if use_data:        # text prompts with ground truths: every rank reads the same un-sharded pipeline
        from b200fw.data.pipeline import GSM8KDataPipeline
        recs = [{"question": f"{i}+1?", "answer": f"#### {i + 1}"} for i in range(16)]
        data = GSM8KDataPipeline(records=recs, prompt_template="plain", max_prompt_tokens=8)
    o = DisaggOrchestrator(cfg, trainer, engine, data=data).initialize()
    if mode_arg.endswith("+leave"):
        # one iteration together; then the last rank shuts down between iterations and the others, once their
        # watcher has seen it, refuse to start the next iteration
        import time
        from b200fw.dist import PeerLostError
        assert o.heartbeat is not None
        o.run()
        if rank == world - 1:
            o.shutdown()
            time.sleep(4.0)
            return {"left": True}
        deadline = time.time() + 20
        while o.heartbeat.lost is None and time.time() < deadline:
            time.sleep(0.02)
        t0 = time.time()
        try:
            o.run()
        except PeerLostError as e:
            return {"lost": e.rank, "reason": e.reason, "took": time.time() - t0, "iterations": len(o.metrics)}
        return {"lost": None}
    if mode_arg.endswith("+fail"):
        # the last rank's engine breaks in the second iteration: every rank must leave the loop with that error
        if rank == world - 1:
            real, calls = o.infer_engine.generate, []

            def broken(*a, **k):
                calls.append(1)
                if len(calls) == 2:
                    raise ValueError("engine lost its KV pool")
                return real(*a, **k)
            o.infer_engine.generate = broken
        try:
            o.run()
        except RuntimeError as e:
            return {"error": str(e), "iterations": len(o.metrics)}
        return {"error": None, "iterations": len(o.metrics)}
    o.run()
    s = o.get_summary()
    if use_data:
        s["reward_fn"] = type(o.reward_fn).__name__
        s["reward_total"] = o.reward_fn.total
    if not o.is_trainer:
        from b200fw.model.hf_io import hf_named_tensors
        s["checksum"] = float(sum(v.double().sum() for _, v in hf_named_tensors(o.infer_engine.model)))
    else:
        with o.train_engine.optimizer.eval_mode():
            from b200fw.model.hf_io import hf_named_tensors
            s["checksum"] = float(sum(v.double().sum() for _, v in hf_named_tensors(o.train_engine.model)))
    return s


def test_disaggregated_loop_with_a_text_dataset_and_the_rule_reward():
    from _dist_util import run_ranks
    res = run_ranks(_disagg_worker, 4, "pipeline+data", timeout=600)
    assert all(r["weights_version"] == r["iterations"] for r in res)
    assert len({round(r["checksum"], 6) for r in res}) == 1
    assert all(r["reward_fn"] == "GSM8KRewardFunction" for r in res)
    # each trainer scored its half of 2 iterations x 4 prompts x 2 samples; rollout ranks score nothing
    assert [r["reward_total"] for r in res] == [8, 8, 0, 0]


def test_disaggregated_loop_two_trainers_two_engines():
    from _dist_util import run_ranks
    for mode in ("sequential", "pipeline"):
        res = run_ranks(_disagg_worker, 4, mode, timeout=600)
        assert [r["role"] for r in res] == ["trainer", "trainer", "rollout", "rollout"]
        assert all(r["weights_version"] == r["iterations"] for r in res)
        # after the final sync every engine holds exactly the trainers' weights
        assert len({round(r["checksum"], 6) for r in res}) == 1, [r["checksum"] for r in res]
        assert res[0]["final_loss"] is not None
        # overlap: back-to-back phases hide nothing; pipelined phases hide the shorter one
        assert (res[0]["avg_overlap_ratio"] == 0.0) == (mode == "sequential"), (mode, res[0]["avg_overlap_ratio"])


def test_a_failed_rollout_rank_ends_the_loop_on_every_rank_with_its_error():
    """One rollout rank's engine raises in the second iteration.  The error travels with the sample exchange: every
    rank raises it at the same point of the same iteration, none is left waiting in a collective."""
    from _dist_util import run_ranks
    for mode in ("sequential+fail", "pipeline+fail"):
        res = run_ranks(_disagg_worker, 4, mode, timeout=300)
        assert all(r["error"] and "rank 3 failed" in r["error"] and "KV pool" in r["error"] for r in res), res
        assert {r["iterations"] for r in res} == {1}, res


def test_clock_sampler_reads_the_median_clock_and_the_active_reasons(tmp_path, monkeypatch):
    """The sampler against a stand-in ``nvidia-smi`` (a script on PATH that prints the query's CSV lines): the median SM
    clock, the maximum, the reasons that were active in any sample; malformed lines are passed over; without the tool
    the summary says so.  Nothing of the GPU's state is written by the sampler: it only runs the query."""
    import os
    import stat
    import time
    from b200fw.obs.clocks import ClockSampler, clocks_during
    fake = tmp_path / "nvidia-smi"
    fake.write_text("#!/bin/sh\n"
                    "case \"$*\" in *--query-gpu=clocks.sm,clocks.max.sm*-lms*) ;; *) echo unexpected args >&2; exit 3;; esac\n"
                    "echo '1300, 1965, Not Active, Not Active, Not Active, Active'\n"
                    "echo '[N/A], 1965, Not Active, Not Active, Not Active, Not Active'\n"
                    "echo 'garbage'\n"
                    "echo '1900, 1965, Not Active, Not Active, Not Active, Not Active'\n"
                    "echo '1400, 1965, Not Active, Active, Not Active, Active'\n"
                    "sleep 30\n")
    fake.chmod(fake.stat().st_mode | stat.S_IEXEC)
    monkeypatch.setenv("PATH", f"{tmp_path}{os.pathsep}{os.environ['PATH']}")
    with clocks_during(0) as c:
        deadline = time.time() + 5
        while len(c.sampler.samples) < 5 and time.time() < deadline:
            time.sleep(0.02)
    assert c.summary == {"sm_mhz": 1400.0, "sm_max_mhz": 1965.0, "reasons": ["hw_thermal_slowdown", "sw_power_cap"],
                         "samples": 3}
    assert c.sampler.proc.poll() is not None                    # the child it started is gone
    monkeypatch.setenv("PATH", str(tmp_path / "empty"))
    s = ClockSampler(0)
    s.start()
    assert s.stop() == {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}


def test_compute_profiler_layer_timing_and_memory_manager_thresholds(monkeypatch):
    """Per-layer timing (context manager and forward hooks on the top-level layers of a model), its report / summary /
    reset; the memory manager's warn / critical thresholds against a stand-in for the device's free-memory query (a
    critical reading empties the allocator's cache and the reserve can be handed back exactly once)."""
    import time
    import torch
    from b200fw.model import ModelConfig, ParallelTransformerModel
    from b200fw.obs import ComputeProfiler, MemoryManager
    prof = ComputeProfiler()
    with prof.profile_layer("sleep"):
        time.sleep(0.01)
    assert prof.layer_ms["sleep"][0] >= 9.0
    off = ComputeProfiler(enabled=False)
    with off.profile_layer("x"):
        pass
    assert not off.layer_ms
    mc = ModelConfig(vocab_size=64, hidden_size=32, num_layers=2, num_heads=2, num_kv_heads=2, head_dim=16,
                     intermediate_size=48, max_position_embeddings=64, tie_word_embeddings=True)
    m = ParallelTransformerModel(mc)
    m.init_weights(0)
    ids = torch.randint(0, 64, (2, 16))
    means = prof.profile_model(m, lambda: m(ids), warmup=1, iters=2)
    assert {"layers.0", "layers.1", "norm"} <= set(means) and all(v > 0 for v in means.values())
    assert "sleep" not in means                                      # the warm-up cleared earlier samples
    assert all(len(v) == 2 for v in prof.layer_ms.values())         # warm-up runs are not counted
    assert not m.layers[0]._forward_hooks and not m.layers[0]._forward_pre_hooks      # hooks removed again
    rep = prof.report()
    assert "layers.0" in rep and "%" in rep
    summ = prof.get_summary()
    assert summ["layers"]["layers.1"]["count"] == 2 and summ["peak_tflops"] == prof.peak_tflops
    assert {p.layer_name for p in prof.layer_profiles} == set(means)
    prof.reset()
    assert not prof.layer_ms and prof.report().count("\n") == 1
    # ---- memory manager ----
    mm = MemoryManager(warn=0.5, critical=0.8)
    assert mm.check() == "ok" or torch.cuda.is_available()          # no device: utilisation reads 0
    free = {"v": 90}
    emptied = []
    monkeypatch.setattr(torch.cuda, "mem_get_info", lambda dev=None: (free["v"], 100))
    monkeypatch.setattr(torch.cuda, "empty_cache", lambda: emptied.append(1))
    mm.enabled = True
    assert mm.check() == "ok" and not mm.events
    free["v"] = 40
    assert mm.check() == "warn" and mm.events == ["warn 0.600"] and not emptied
    free["v"] = 10
    assert mm.check() == "critical" and mm.events[-1] == "critical 0.900" and emptied == [1]
    mm._reserve = object()
    assert mm.release_reserve() is True and mm.release_reserve() is False and len(emptied) == 3
    ref_form = MemoryManager("cpu", warning_threshold=0.7, critical_threshold=0.9)
    assert (ref_form.warn, ref_form.critical) == (0.7, 0.9)
    ref_form.enabled = False
    assert ref_form.get_stats() == {} and ref_form.check_memory_pressure()["utilization"] == 0
    ref_form.reserve_buffer(1)
    ref_form.release_buffer()


def test_disaggregated_ranks_do_not_start_an_iteration_once_a_peer_has_left():
    from _dist_util import run_ranks
    res = run_ranks(_disagg_worker, 4, "sequential+leave", timeout=300)
    assert res[3] == {"left": True}
    for r in res[:3]:
        assert r["lost"] == 3 and "shutdown" in r["reason"] and r["took"] < 0.5, r
