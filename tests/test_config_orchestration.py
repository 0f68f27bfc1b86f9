"""Config loading / validation, the colocate loop (native, mock and mocked-vLLM back ends), weight sync
paths, and host-side fault injection."""
import asyncio
import glob
import json
import math
import os
import tempfile
import threading

import pytest
import torch

from b200fw.config import (ColocateConfig, build_colocate_config, get_nested, load_yaml_config,
                           validate_parallel_config)
from b200fw.orch import ColocateOrchestrator, OrchestratorState
from b200fw.sync import (DeltaComputer, DoubleBufferedLoRA, IPCWeightTransfer, PeerWeightSync, SwiftSyncConfig, SwiftSyncTransfer,
                         VLLMClient, WeightUpdateManager, classify_error, fletcher_checksum)

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_yaml_mapping_overrides_and_unknown_keys():
    y = {"model": {"name_or_path": "/m", "max_seq_len": 512}, "runtime": {"tp_size": 2, "dp_size": 4, "precision": "fp32"},
         "distributed": {"pp_size": 1, "zero_stage": 3}, "training": {"mode": "sft", "batch_size": 8},
         "lora": {"rank": 0, "dropout": 0.1}, "inference_preview": {"max_tokens": 9}, "bogus": {"key": 1}}
    cfg, unknown = build_colocate_config(y, {"total_iterations": 3, "learning_rate": None})
    assert (cfg.model_path, cfg.max_seq_len, cfg.tp_size, cfg.dp_size, cfg.amp_dtype) == ("/m", 512, 2, 4, "fp32")
    assert cfg.zero_stage == 3            # distributed.zero_stage is honoured when training.zero_stage is absent
    assert cfg.max_tokens == 9 and cfg.total_iterations == 3 and cfg.learning_rate == 1e-5
    assert unknown == ["bogus.key"]
    y["training"]["zero_stage"] = 2
    assert build_colocate_config(y)[0].zero_stage == 2
    assert get_nested(y, "runtime.tp_size") == 2 and get_nested(y, "a.b", 7) == 7
    with pytest.raises(KeyError):
        build_colocate_config({}, {"nope": 1})


def test_deterministic_switch_is_read_from_yaml_and_applied(tmp_path):
    from b200fw.config import apply_determinism
    y = tmp_path / "c.yaml"
    y.write_text("runtime:\n  deterministic: true\n  seed: 11\n")
    cfg, unknown = build_colocate_config(load_yaml_config(str(y)))
    assert cfg.deterministic is True and cfg.seed == 11 and unknown == []
    was = os.environ.get("B200FW_DETERMINISTIC")
    try:
        apply_determinism(True, 11)
        a = torch.rand(3)
        assert os.environ["B200FW_DETERMINISTIC"] == "1" and torch.are_deterministic_algorithms_enabled()
        apply_determinism(True, 11)
        assert torch.equal(a, torch.rand(3))                      # same seed, same draws
        apply_determinism(False)
        assert "B200FW_DETERMINISTIC" not in os.environ and not torch.are_deterministic_algorithms_enabled()
    finally:
        apply_determinism(False)
        if was is not None:
            os.environ["B200FW_DETERMINISTIC"] = was


def test_reward_values_come_from_yaml(tmp_path):
    y = tmp_path / "c.yaml"
    y.write_text("reward:\n  type: gsm8k_rule\n  correct_reward: 2.0\n  format_reward: -0.25\n  wrong_reward: -3.0\n"
                 "experiment:\n  stage: rl\nruntime:\n  device: auto\n")
    cfg, unknown = build_colocate_config(load_yaml_config(str(y)))
    assert (cfg.reward_correct, cfg.reward_format, cfg.reward_wrong) == (2.0, -0.25, -3.0) and unknown == []
    from b200fw.reward import GSM8KRewardFunction
    rf = GSM8KRewardFunction(correct=cfg.reward_correct, wrong=cfg.reward_format, no_answer=cfg.reward_wrong)
    assert rf([["#### 4", "#### 5", "dunno"]], [4]) == [[2.0, -0.25, -3.0]]


def test_parallel_validation_rules():
    ok = ColocateConfig(tp_size=2, dp_size=2, pp_size=2, num_micro_batches=2, batch_size=8, zero_stage=1, training_mode="sft")
    validate_parallel_config(ok, 8)
    for bad, world in ((dict(tp_size=2), 8), (dict(num_micro_batches=1), 8), (dict(batch_size=6), 8),
                       (dict(zero_stage=2), 8), (dict(training_mode="grpo"), 8), (dict(amp_dtype="int8"), 8)):
        c = ColocateConfig(**{**dict(tp_size=2, dp_size=2, pp_size=2, num_micro_batches=2, batch_size=8, zero_stage=1,
                                     training_mode="sft"), **bad})
        with pytest.raises(ValueError):
            validate_parallel_config(c, world if "tp_size" not in bad else 16)


def test_yaml_values_are_brought_to_their_field_types(tmp_path):
    """YAML reads ``1e-5`` (no dot) as a string and ``8.0`` as a float; command lines hand over strings.  Each value is
    converted to its field's type, and one that cannot be is refused with the key in the message."""
    y = tmp_path / "c.yaml"
    y.write_text("training:\n  learning_rate: 1e-5\n  batch_size: 8.0\n  mode: sft\n"
                 "runtime:\n  tp_size: '2'\n  sequence_parallel: 'yes'\n"
                 "lora:\n  target_modules: q_proj, v_proj\n  rank: 0\n")
    cfg, unknown = build_colocate_config(load_yaml_config(str(y)), overrides={"max_grad_norm": "0.5", "dp_size": "1"})
    assert unknown == []
    assert cfg.learning_rate == 1e-5 and isinstance(cfg.learning_rate, float)
    assert cfg.batch_size == 8 and isinstance(cfg.batch_size, int)
    assert cfg.tp_size == 2 and cfg.sequence_parallel is True and cfg.max_grad_norm == 0.5 and cfg.dp_size == 1
    assert cfg.lora_target_modules == ["q_proj", "v_proj"] and cfg.lora_rank == 0
    for text, key in (("training:\n  learning_rate: fast\n", "training.learning_rate"),
                      ("training:\n  batch_size: 2.5\n", "training.batch_size"),
                      ("runtime:\n  sequence_parallel: maybe\n", "runtime.sequence_parallel"),
                      ("runtime:\n  tp_size: [2]\n", "runtime.tp_size")):
        y.write_text(text)
        with pytest.raises(ValueError, match=key.replace(".", r"\.")):
            build_colocate_config(load_yaml_config(str(y)))
    for bad in (dict(tp_size=0), dict(batch_size=0), dict(gradient_accumulation_steps=0), dict(learning_rate=float("nan")),
                dict(learning_rate=-1.0), dict(zero_stage=4), dict(lora_rank=-1), dict(max_seq_len=1)):
        with pytest.raises(ValueError, match=next(iter(bad))):
            validate_parallel_config(ColocateConfig(**bad), 1)


def test_every_shipped_config_parses_and_validates():
    n = 0
    for f in glob.glob(os.path.join(ROOT, "configs", "**", "*.yaml"), recursive=True):
        y = load_yaml_config(f)
        if "training" not in y:
            continue
        cfg, unknown = build_colocate_config(y)
        assert unknown == [], (f, unknown)
        validate_parallel_config(cfg, cfg.tp_size * cfg.dp_size * cfg.pp_size)
        n += 1
    assert n > 40


def _run(cfg, **kw):
    async def go():
        o = ColocateOrchestrator(cfg, **kw)
        await o.initialize()
        await o.run()
        s = o.get_summary()
        await o.shutdown()
        return o, s
    return asyncio.run(go())


def _tiny_cfg(tmp, **over):
    base = dict(model_preset="tiny128", training_mode="grpo", total_iterations=3, batch_size=2, num_samples_per_prompt=2,
                max_tokens=6, max_seq_len=64, lora_rank=0, grpo_beta=0.01, gradient_accumulation_steps=1, amp_dtype="fp32",
                inference_backend="native", synthetic_data=True, synthetic_prompt_len=12, max_data_samples=64,
                kv_num_blocks=64, warmup_steps=0, output_dir=os.path.join(tmp, "out"),
                checkpoint_save_dir=os.path.join(tmp, "ckpt"), tensorboard=False, learning_rate=1e-3)
    base.update(over)
    return ColocateConfig(**base)


def test_colocate_grpo_native_engine_full_loop():
    with tempfile.TemporaryDirectory() as d:
        cfg = _tiny_cfg(d, icepop_enabled=True, c3po_plus_enabled=True, c3po_plus_token_budget=4,
                        c3po_plus_target_batch_tokens=64, checkpoint_save_interval=2)
        o, s = _run(cfg)
        assert o.state == OrchestratorState.DONE and s["results"]["failed_iterations"] == 0
        assert s["results"]["final_weights_version"] == 3 and s["weight_sync"]["transfers"] == 3
        per_iter = ["inferring", "rewarding", "training", "sleeping", "syncing"]
        assert o.state_log[:5] == per_iter and o.state_log[-1] == "done"
        assert all(m.tokens_generated > 0 and m.train_metrics.grad_norm > 0 for m in o.metrics)
        out = cfg.output_dir
        for name in ("config_snapshot.json", "run_summary.json", "metrics_rank0.jsonl", "loss_curve.csv",
                     "memory_report.json", "memory_timeline_rank0.json"):
            assert os.path.exists(os.path.join(out, name)), name
        rows = [json.loads(l) for l in open(os.path.join(out, "metrics_rank0.jsonl"))]
        assert len(rows) == 3 and {"loss", "avg_reward", "t_training", "weights_version"} <= set(rows[0])
        assert {"iter_2", "latest", "final"} <= set(os.listdir(cfg.checkpoint_save_dir))
        # the rollout engine really follows the trainer: after the last sync its weights equal the export
        from b200fw.model.hf_io import hf_named_tensors
        want = o.train_engine.export_weights()
        got = dict(hf_named_tensors(o.infer_engine.model))
        assert all(torch.equal(want[k], got[k]) for k in want)


def test_colocate_lora_swiftsync_and_async_pipeline_staleness():
    with tempfile.TemporaryDirectory() as d:
        cfg = _tiny_cfg(d, lora_rank=4, swift_sync_enabled=True, swift_sync_fallback_full_every=2,
                        async_pipeline_enabled=True, async_pipeline_max_staleness=1, total_iterations=4,
                        checkpoint_save_enabled=False)
        o, s = _run(cfg)
        assert s["results"]["failed_iterations"] == 0
        sw = s["swift_sync"]
        assert sw["full_syncs"] >= 2 and sw["delta_syncs"] >= 1 and sw["version"] == 4
        assert max(m.rollout_staleness for m in o.metrics) <= 1


def _tp_colocate_worker(rank, world, tmp, async_pipeline):
    cfg = _tiny_cfg(os.path.join(tmp, f"r{rank}"), tp_size=world, total_iterations=2, batch_size=2, num_samples_per_prompt=2,
                    sequence_parallel=True, checkpoint_save_enabled=False, async_pipeline_enabled=async_pipeline,
                    async_pipeline_max_staleness=1)
    o, s = _run(cfg)
    eng = o.infer_engine
    from b200fw.model.hf_io import hf_named_tensors
    full = {k: v.clone() for k, v in o.train_engine.export_weights().items()}
    mine = dict(hf_named_tensors(eng.model))
    same = all(torch.equal(full[k], mine[k]) for k in full)
    ro = o._rollout(o._next_batch())
    return (eng.config.inference_mode, eng.model.tp_size, same, ro.responses, s["results"]["completed_iterations"],
            [m.error for m in o.metrics], eng.stats["decode_tokens"] + eng.stats["prefill_tokens"])


def test_tensor_parallel_grpo_uses_native_rollouts_shared_over_the_tp_group():
    """TP 2: every rank serves rollouts from a full single-GPU copy of the policy (not the mock engine), the two
    ranks split the prompts and end up with the same responses; the copy tracks the trained weights."""
    from _dist_util import run_ranks
    for async_pipeline in (False, True):
        with tempfile.TemporaryDirectory() as d:
            res = run_ranks(_tp_colocate_worker, 2, d, async_pipeline, timeout=600)
        for mode, tp, same, responses, done, errors, work in res:
            assert mode == "kv_cache" and tp == 1 and same and done == 2 and errors == [None, None] and work > 0
        assert res[0][3] == res[1][3] and len(res[0][3]) == 2 and len(res[0][3][0]) == 2     # identical [B][K] token lists


def _dp_colocate_worker(rank, world, tmp, stage):
    cfg = _tiny_cfg(os.path.join(tmp, f"r{rank}"), dp_size=world, zero_stage=stage, total_iterations=2, batch_size=4,
                    num_samples_per_prompt=2, checkpoint_save_enabled=False)
    o, s = _run(cfg)
    from b200fw.model.hf_io import hf_named_tensors
    want = o.train_engine.export_weights()
    got = dict(hf_named_tensors(o.infer_engine.model))
    return (s["results"]["failed_iterations"], all(torch.equal(want[k], got[k]) for k in want),
            float(sum(v.double().sum() for v in want.values())), [b.prompt_indices for b in [o._next_batch()]])


def test_colocate_data_parallel_with_sharded_optimizer_states_and_parameters():
    """DP 2 with ZeRO-2 and ZeRO-3 (parameters released between steps): the rollout copy is built from the gathered
    weights, follows the trainer, the ranks stay in step and draw different prompts."""
    from _dist_util import run_ranks
    for stage in (2, 3):
        with tempfile.TemporaryDirectory() as d:
            res = run_ranks(_dp_colocate_worker, 2, d, stage, timeout=600)
        assert [r[0] for r in res] == [0, 0] and all(r[1] for r in res), stage
        assert res[0][2] == res[1][2] and res[0][3] != res[1][3], stage


def test_summary_without_iterations_and_state_transition_coroutine():
    o = ColocateOrchestrator(ColocateConfig(model_preset="tiny128"))
    assert o.get_summary() == {"status": "no_data"} and o.state == OrchestratorState.INIT
    asyncio.run(o._transition(OrchestratorState.TRAINING))
    assert o.state == OrchestratorState.TRAINING and o.state_log[-1] == "training"


def test_colocate_sft_mode_and_resume():
    with tempfile.TemporaryDirectory() as d:
        cfg = _tiny_cfg(d, training_mode="sft", inference_preview_enabled=False, total_iterations=3)
        o, s = _run(cfg)
        assert s["results"]["final_loss"] is not None and o.state_log.count("training") == 3
        # with the preview on, every iteration also generates one sample from the freshly synced weights
        cfgp = _tiny_cfg(os.path.join(d, "p"), training_mode="sft", inference_preview_enabled=True, total_iterations=2,
                         checkpoint_save_enabled=False)
        op, _ = _run(cfgp)
        assert op.state_log.count("inferring") == 2 and op.last_preview is not None
        assert all(0 < m.tokens_generated <= cfgp.max_tokens and "inferring" in m.state_durations for m in op.metrics)
        assert op.infer_engine.weights_version >= 2
        cfg2 = _tiny_cfg(d, training_mode="sft", inference_preview_enabled=False, total_iterations=1,
                         resume_from=os.path.join(cfg.checkpoint_save_dir, "final"))
        o2, _ = _run(cfg2)
        assert o2.train_engine.step_count == 4


def test_eval_before_after_artifacts_and_fixed_prompt_comparison():
    import json
    from b200fw.data.pipeline import GSM8KDataPipeline
    recs = [{"question": f"{i} plus {i}?", "answer": f"#### {2 * i}"} for i in range(8)]
    with tempfile.TemporaryDirectory() as d:
        cfg = _tiny_cfg(d, training_mode="sft", inference_preview_enabled=False, total_iterations=2, synthetic_data=False,
                        eval_num_prompts=2, eval_max_tokens=4, checkpoint_save_enabled=False, tensorboard=True)
        data = GSM8KDataPipeline(records=recs, prompt_template="plain")
        o, s = _run(cfg, data=data)
        out = cfg.output_dir
        before = json.load(open(os.path.join(out, "eval_before.json")))
        after = json.load(open(os.path.join(out, "eval_after.json")))
        cmp_ = json.load(open(os.path.join(out, "fixed_prompt_comparison.json")))
        for payload, stage in ((before, "before"), (after, "after")):
            m = payload["metrics"]
            assert m["stage"] == stage and m["num_samples"] == 2 and m["eval_loss"] > 0
            assert abs(m["perplexity"] - math.exp(min(m["eval_loss"], 20.0))) < 1e-6
            assert 0.0 <= m["token_f1"] <= 1.0 and 0.0 <= m["bleu4"] <= 1.0 and 0.0 <= m["exact_match"] <= 1.0
            assert [x["index"] for x in payload["samples"]] == [0, 1]
            assert all(x["generated_tokens"] <= 4 and x["reference"].startswith("####") for x in payload["samples"])
        assert before["metrics"]["step"] == 0 and after["metrics"]["step"] == 2
        assert after["metrics"]["eval_loss"] < before["metrics"]["eval_loss"]          # the same two prompts were trained on
        assert [r["prompt"] for r in cmp_["samples"]] == [x["prompt"] for x in before["samples"]]
        assert set(cmp_["samples"][0]) >= {"before_generated", "after_generated", "before_token_f1", "after_exact_match"}
        assert s["eval"]["before"]["num_samples"] == 2 and "after" in s["eval"]
        res = s["results"]
        assert res["completed_iterations"] == 2 and res["total_time_s"] >= res["avg_iteration_time_s"] > 0
        assert set(s["stage_avg_durations"]) == set(s["stage_averages"]) and "peak_mb" in s["memory"]
        assert "timers" in s["metrics_summary"] and o.metrics_history is o.metrics
        rs = json.load(open(os.path.join(out, "run_summary.json")))
        assert rs["status"] == "completed" and rs["mode"] == "sft" and rs["run"]["output_dir"] == out
        assert rs["run"]["ended_at_unix"] >= rs["run"]["started_at_unix"] > 0
        assert rs["artifacts"]["eval_before"].endswith("eval_before.json") and "metrics_jsonl" in rs["artifacts"]
        perf = rs["performance"]
        assert perf["world_size"] == 1 and perf["global_batch_size"] == cfg.batch_size and perf["avg_step_time_s"] > 0
        assert perf["tokens_per_second"] > 0 and perf["model_arch"]["vocab_size"] == 8192
        # a tiny model on a CPU is a vanishing fraction of the B200 peak: the rounded percentage may be 0.00
        assert 0 <= perf["mfu_percent"] < 100 and perf["per_gpu_training_flops"] > 0 and perf["actual_tflops_per_gpu"] >= 0
        assert perf["primary_metric"] == "mfu" and perf["model_params"] > 0
        from b200fw.obs import read_scalars
        tags = read_scalars(os.path.join(out, "tensorboard"))
        assert "eval/before_loss" in tags and "eval/after_token_f1" in tags and "train/loss" in tags
        assert os.path.exists(os.path.join(out, "loss_curve.csv"))
    with tempfile.TemporaryDirectory() as d:                                            # eval.num_prompts: 0 -> no files
        cfg = _tiny_cfg(d, training_mode="sft", inference_preview_enabled=False, total_iterations=1,
                        checkpoint_save_enabled=False)
        _run(cfg)
        assert not os.path.exists(os.path.join(cfg.output_dir, "eval_before.json"))


class _FakeResp:
    def __init__(self, payload=None):
        self.payload, self.status_code = payload or {}, 200

    def raise_for_status(self):
        pass

    def json(self):
        return self.payload


class _FakeHttp:
    """Stand-in for the vLLM HTTP server: records calls, can fail the first N wake-ups."""

    def __init__(self, fail_wake=0, fail_update=False):
        self.calls, self.fail_wake, self.fail_update, self.bodies = [], fail_wake, fail_update, []

    async def post(self, url, **kw):
        self.bodies.append((url, kw))
        self.calls.append(url.split("/")[-1].split("?")[0])
        if "wake_up" in url and self.fail_wake > 0:
            self.fail_wake -= 1
            raise ConnectionError("server busy")
        if "update_weights" in url and self.fail_update:
            raise ValueError("bad payload")
        if url.endswith("/v1/completions"):
            body = kw["json"]
            return _FakeResp({"choices": [{"text": f"Step 1: think\n#### {7 + i}"} for i in range(body["n"])]})
        return _FakeResp()

    async def get(self, url, **kw):
        self.calls.append("health")
        return _FakeResp()


def test_vllm_client_retry_taxonomy_and_ipc_chunking():
    assert classify_error(ValueError()) == "fatal" and classify_error(RuntimeError("CUDA out of memory")) == "oom"
    assert classify_error(ConnectionError()) == "retry"
    http = _FakeHttp(fail_wake=2)
    c = VLLMClient("http://x", max_retries=3, backoff_s=0.0, client=http)
    asyncio.run(c.wake_up())
    assert http.calls.count("wake_up") == 3
    state = {f"w{i}": torch.randn(4, 4) for i in range(10)}
    http = _FakeHttp()
    ipc = IPCWeightTransfer(VLLMClient("http://x", backoff_s=0.0, client=http), chunk_size=4)
    assert [len(c) for c in ipc._chunk_handles(ipc.build_ipc_handles(state))] == [4, 4, 2]
    asyncio.run(ipc.push_weights(state))
    assert http.calls == ["reset_prefix_cache", "sleep", "init_weight_transfer_engine", "start_weight_update",
                          "update_weights", "update_weights", "update_weights", "finish_weight_update", "wake_up"]
    # request shapes of the vLLM control protocol: relative paths, query parameters, JSON bodies
    by_path = {u: kw for u, kw in http.bodies}
    assert by_path["/sleep"] == {"params": {"level": 1}} and by_path["/wake_up"] == {}
    assert by_path["/reset_prefix_cache"]["params"] == {"reset_running_requests": False, "reset_external": False}
    assert by_path["/start_weight_update"] == {"json": {"is_checkpoint_format": True}}
    assert set(by_path["/update_weights"]["json"]["update_info"]) == {"names", "shapes", "dtypes", "ipc_handles"}
    assert by_path["/init_weight_transfer_engine"] == {"json": {"init_info": {}}} and by_path["/finish_weight_update"] == {"json": {}}
    c2 = VLLMClient("http://x", backoff_s=0.0, client=_FakeHttp(), retry_delay=0.0)
    assert asyncio.run(c2.wake_up(tags=["weights", "kv_cache"])) is True and asyncio.run(c2.health_check()) is True
    assert c2._client.bodies[0] == ("/wake_up", {"params": {"tags": ["weights", "kv_cache"]}})
    # a non-retriable failure mid-transfer still wakes the server up, then re-raises
    http = _FakeHttp(fail_update=True)
    ipc = IPCWeightTransfer(VLLMClient("http://x", backoff_s=0.0, client=http), chunk_size=4)
    with pytest.raises(ValueError):
        asyncio.run(ipc.push_weights(state))
    assert http.calls[-1] == "wake_up" and ipc.stats.failures == 1
    assert len(IPCWeightTransfer.checksum(state)) == 32


def test_colocate_grpo_with_a_vllm_server_for_rollouts_and_ipc_weight_push():
    """inference_backend "vllm": completions over HTTP (K per prompt), rule reward on the text, training on the
    re-tokenised responses, then sleep -> weight push in chunks -> wake."""
    from b200fw.data.pipeline import GSM8KDataPipeline
    recs = [{"question": f"{i} plus 7?", "answer": f"#### {7 + (i % 2)}"} for i in range(8)]
    http = _FakeHttp()
    with tempfile.TemporaryDirectory() as d:
        cfg = _tiny_cfg(d, inference_backend="vllm", synthetic_data=False, total_iterations=2, batch_size=2,
                        num_samples_per_prompt=2, checkpoint_save_enabled=False, max_seq_len=128)
        o, s = _run(cfg, data=GSM8KDataPipeline(records=recs, prompt_template="plain"),
                    vllm_client=VLLMClient("http://x", backoff_s=0.0, client=http))
    assert o.infer_engine is None and s["results"]["completed_iterations"] == 2 and s["results"]["failed_iterations"] == 0
    comps = [kw["json"] for u, kw in http.bodies if u == "/v1/completions"]
    assert len(comps) == 4 and all(c["n"] == 2 and c["max_tokens"] == cfg.max_tokens and "plus 7?" in c["prompt"] for c in comps)
    assert http.calls.count("sleep") == 2 and http.calls.count("update_weights") >= 2 and http.calls.count("wake_up") >= 2
    # responses "#### 7" / "#### 8" against answers 7 / 8: some right (+1), the rest well formed but wrong (-0.5)
    assert {m.avg_reward for m in o.metrics} <= {1.0, 0.25, -0.5} and all(m.train_metrics is not None for m in o.metrics)
    assert all(m.tokens_generated > 0 for m in o.metrics) and o.weights_version == 2


def _tp_vllm_worker(rank, world, tmp):
    from b200fw.data.pipeline import GSM8KDataPipeline
    recs = [{"question": f"{i} plus 7?", "answer": f"#### {7 + (i % 2)}"} for i in range(8)]
    http = _FakeHttp()
    cfg = _tiny_cfg(os.path.join(tmp, f"r{rank}"), inference_backend="vllm", synthetic_data=False, total_iterations=1,
                    batch_size=2, num_samples_per_prompt=2, checkpoint_save_enabled=False, max_seq_len=128, tp_size=world,
                    sequence_parallel=True)
    o, s = _run(cfg, data=GSM8KDataPipeline(records=recs, prompt_template="plain"),
                vllm_client=VLLMClient("http://x", backoff_s=0.0, client=http))
    return (http.calls.count("completions"), s["results"]["failed_iterations"], o.metrics[0].avg_reward,
            o.metrics[0].train_metrics.loss)


def test_vllm_rollouts_are_queried_once_per_tensor_parallel_group():
    from _dist_util import run_ranks
    with tempfile.TemporaryDirectory() as d:
        res = run_ranks(_tp_vllm_worker, 2, d, timeout=600)
    assert [r[0] for r in res] == [2, 0] and [r[1] for r in res] == [0, 0]      # rank 0 asked, rank 1 received
    assert res[0][2] == res[1][2] and abs(res[0][3] - res[1][3]) < 1e-6         # same rewards, same loss


def test_weight_update_manager_rolls_back():
    m = torch.nn.Linear(4, 4)
    mgr = WeightUpdateManager(m)
    before = m.weight.detach().clone()
    assert mgr.update_weights({"weight": torch.ones(4, 4)}) and mgr.version == 1
    assert not mgr.update_weights({"weight": torch.ones(4, 4) * 2, "bias": torch.full((4,), float("nan"))})
    assert torch.equal(m.weight, torch.ones(4, 4)) and mgr.rollbacks == 1 and mgr.version == 1
    assert not mgr.update_weights({"weight": torch.ones(3, 3)})
    assert not torch.equal(before, m.weight.detach())


def test_swift_sync_delta_math_policy_and_double_buffer():
    dc = DeltaComputer(fallback_full_every=3)
    s0 = {"a": torch.ones(3)}
    assert torch.equal(dc.compute_delta(s0)["a"], torch.ones(3))           # first call: full state
    assert torch.equal(dc.compute_delta({"a": torch.full((3,), 1.5)})["a"], torch.full((3,), 0.5))
    assert [dc.should_full_sync(i) for i in range(7)] == [False, False, False, True, False, False, True]
    db = DoubleBufferedLoRA({"a": torch.zeros(2)})
    db.apply_delta_to_shadow({"a": torch.ones(2)})
    assert torch.equal(db.get_active_state()["a"], torch.zeros(2))           # not visible before the swap
    assert db.swap_buffers() == 1 and torch.equal(db.get_active_state()["a"], torch.ones(2))
    db.apply_delta_to_shadow({"a": torch.ones(2)})                           # shadow was levelled after the swap
    db.swap_buffers()
    assert torch.equal(db.get_active_state()["a"], torch.full((2,), 2.0)) and db.version == 2

    class W:
        def __init__(self):
            self.seen = []

        def update_weights(self, state, mode="full"):
            self.seen.append(mode)

    w = W()
    t = SwiftSyncTransfer(w)
    t.sync_full({"a": torch.zeros(2)})
    t.sync_delta({"a": torch.ones(2)})
    assert w.seen == ["full", "delta"] and t.get_stats()["version"] == 2 and t.stats.bytes_sent == 16
    t2 = SwiftSyncTransfer(object())                                         # worker without update_weights
    with pytest.raises(AttributeError):
        t2.sync_delta({"a": torch.ones(2)})
    assert t2.buffer.version == 0


def test_swift_sync_single_buffer_mode_async_full_and_stateless_delta():
    class W:
        def __init__(self):
            self.modes = []

        async def update_weights(self, state, mode="delta"):
            self.modes.append(mode)
    t = SwiftSyncTransfer(SwiftSyncConfig(enabled=True, enable_double_buffer=False))      # config first, as the reference
    t.initialize({"A": torch.zeros(2, 2)})
    assert t.version == 0 and t.double_buffer is None and t.initialized
    w = W()
    assert t.sync_delta({"A": torch.ones(2, 2)}, w) == 1                                   # async worker from sync code
    assert torch.equal(t.buffer.get_active_state()["A"], torch.ones(2, 2))                 # updated in place
    assert asyncio.run(t.sync_full_async({"A": torch.full((2, 2), 9.0)})) == 2
    assert torch.equal(t.prev_snapshot["A"], torch.full((2, 2), 9.0)) and w.modes == ["delta", "full"]
    assert asyncio.run(t.sync_delta_async({"A": torch.ones(2, 2)}, w)) == 3
    assert float(t.buffer.get_active_state()["A"][0, 0]) == 10.0 and t.get_stats_summary()["config"]["enable_double_buffer"] is False

    class NoApi:
        pass
    t2 = SwiftSyncTransfer(SwiftSyncConfig(enabled=True))
    t2.initialize({"A": torch.zeros(2, 2)})
    try:
        t2.sync_delta({"A": torch.ones(2, 2)}, NoApi())
        raise AssertionError("a worker without update_weights must be refused")
    except AttributeError:
        pass
    assert t2.version == 0 and float(t2.buffer.get_active_state()["A"].sum()) == 0.0
    # the reference declares sync_delta / sync_full async: the returned version can be awaited as well
    class SyncW:
        def update_weights(self, state, mode="delta"):
            pass
    r = t2.sync_delta({"A": torch.ones(2, 2)}, SyncW())
    assert r == 1 and isinstance(r, int) and r + 1 == 2 and asyncio.run(r).delta_bytes == 16

    async def awaited():
        return await t2.sync_full({"A": torch.zeros(2, 2)}, SyncW())
    assert asyncio.run(awaited()).version == 2 and t2.version == 2
    c = DeltaComputer(SwiftSyncConfig(enabled=True, fallback_full_every=5))
    assert c.should_full_sync(5) and not c.should_full_sync(0) and not c.should_full_sync(7)
    d = c.compute_delta({"a": torch.ones(1), "b": torch.full((1,), 3.0)}, {"a": torch.zeros(1)})
    assert float(d["a"]) == 1.0 and float(d["b"]) == 3.0 and c._step_count == 1 and c.prev is None


def test_double_buffer_swap_under_threads():
    db = DoubleBufferedLoRA({"a": torch.zeros(8)})
    def work():
        for _ in range(50):
            db.apply_delta_to_shadow({"a": torch.ones(8)})
            db.swap_buffers()
    ts = [threading.Thread(target=work) for _ in range(4)]
    [t.start() for t in ts]
    [t.join() for t in ts]
    assert db.version == 200 and db.swap_count == 200
    a = db.get_active_state()["a"]
    assert torch.all(a == a[0])                                              # never torn


def test_peer_write_refuses_tensors_that_do_not_match_the_layout():
    """Sizes are checked on the host before anything is launched: the device kernel reads as many elements as the
    layout says, so a shorter source must never reach it."""
    ps = PeerWeightSync([("w", (4, 8)), ("b", (8,))], torch.float32, torch.device("cpu"))
    with pytest.raises(ValueError):
        ps.write({"w": torch.ones(4, 7)})
    with pytest.raises(KeyError):
        ps.write({"unknown": torch.ones(8)})
    cks, nbytes = ps.write({"w": torch.ones(32), "b": torch.zeros(8)})          # same count, other shape: accepted
    assert nbytes == 40 * 4 and torch.equal(ps.staging.view("w"), torch.ones(4, 8))


def test_peer_write_checksum_rejects_corruption():
    layout = [("w", (6, 5)), ("b", (7,))]
    ps = PeerWeightSync(layout, torch.bfloat16, torch.device("cpu"))
    got = {}

    class Eng:
        def load_weights(self, views):
            got.update({k: v.clone() for k, v in views.items()})

    state = {"w": torch.randn(6, 5), "b": torch.randn(7)}
    assert ps.sync(True, state, Eng()) == 1 and torch.equal(got["w"], state["w"].to(torch.bfloat16))
    got.clear()
    assert ps.sync(True, {"w": state["w"] * 2, "b": state["b"]}, Eng(), corrupt=True) == 1     # version kept
    assert got == {} and ps.get_stats()["rejected"] == 1
    # a delta (add mode) touches one tensor only; its checksum covers exactly that span and is verified too
    ps.sync(True, state, Eng())                                   # clean image again (version 2)
    got.clear()
    d = {"b": torch.ones(7)}
    assert ps.sync(True, d, Eng(), add=True) == 3
    assert torch.equal(got["b"], (state["b"].to(torch.bfloat16).float() + 1).to(torch.bfloat16))
    got.clear()
    assert ps.sync(True, d, Eng(), add=True, corrupt=True) == 3 and got == {} and ps.get_stats()["rejected"] == 2
    c0, c1 = fletcher_checksum(torch.tensor([1.0, 2.0], dtype=torch.bfloat16))
    assert c0 == 0x3F80 + 0x4000 and c1 == 0x3F80 + 2 * 0x4000


def _nccl_worker(rank, world):
    import torch.distributed as dist
    from b200fw.sync import NCCLWeightTransfer
    dist.init_process_group("gloo", rank=rank, world_size=world)
    t = NCCLWeightTransfer()
    if rank == 0:
        state = {"a": torch.arange(6.0).reshape(2, 3), "b": torch.ones(4)}
        return t.broadcast_weights(state)
    out = t.receive_weights({"a": torch.zeros(2, 3), "b": torch.zeros(4)})
    assert torch.equal(out["a"], torch.arange(6.0).reshape(2, 3)) and t.version == 1
    return t.version


def test_nccl_transfer_baseline_over_gloo():
    from _dist_util import run_ranks
    assert run_ranks(_nccl_worker, 2) == [1, 1]


def _dead_rank_worker(rank, world):
    """Host-side failure: rank 1 never joins the collective; rank 0's bounded wait raises."""
    import datetime
    import torch.distributed as dist
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=3))
    if rank == 1:
        return "left"
    from b200fw.dist.comm import AsyncAllReduce
    h = AsyncAllReduce().launch(torch.ones(4), dist.group.WORLD)
    try:
        h.wait(timeout_sec=1.0)
    except RuntimeError as e:
        return f"detected: {e}"
    return "not detected"


def test_missing_rank_is_detected_by_bounded_wait():
    from _dist_util import run_ranks
    res = run_ranks(_dead_rank_worker, 2)
    assert res[1] == "left" and res[0].startswith("detected")


def test_ray_object_store_transfer_against_a_stand_in_ray(monkeypatch):
    """The object-store backend (CPU copy -> ray.put / ray.get) with a stand-in ``ray`` module: publish bumps the
    version, fetch returns the tensors on the requested device, the manager routes both ends."""
    import sys
    import types
    from b200fw.sync.nccl_transfer import RayObjectStoreTransfer, WeightTransferManager
    store = {}

    def put(obj):
        ref = f"ref{len(store)}"
        store[ref] = obj
        return ref

    monkeypatch.setitem(sys.modules, "ray", types.SimpleNamespace(put=put, get=lambda ref: store[ref]))
    t = RayObjectStoreTransfer()
    assert t.available
    state = {"w": torch.arange(6.0).reshape(2, 3), "b": torch.ones(4)}
    ref = t.publish_weights(state)
    assert ref in store and t.version == 1
    got = t.fetch_weights(device="cpu")
    assert torch.equal(got["w"], state["w"]) and got["w"] is not state["w"]
    loaded = {}

    class Eng:
        def load_weights(self, s):
            loaded.update(s)

    m = WeightTransferManager("ray_object_store")
    assert m.sync_weights(True, state) == 1
    assert m.sync_weights(False, engine=Eng()) == 2 and torch.equal(loaded["b"], state["b"])


def test_swiftsync_low_rank_worker_keeps_engine_equal_to_merged_export(tmp_path):
    """The colocated SwiftSync worker's plan (stacked per-module operands filled by two bulk index copies, one GEMM per
    module) run through the ops' CPU forms: after delta and full syncs the engine's weights equal a fresh merged
    export, the trainer's frozen base never moves."""
    import asyncio
    from b200fw.config import ColocateConfig
    from b200fw.model.hf_io import hf_named_tensors
    from b200fw.model.lora import LinearWithLoRA
    from b200fw.orch import ColocateOrchestrator
    cfg = ColocateConfig(model_preset="tiny", training_mode="grpo", total_iterations=1, batch_size=2,
                         num_samples_per_prompt=2, max_tokens=4, lora_rank=8, lora_alpha=16.0, grpo_beta=0.0,
                         gradient_accumulation_steps=1, zero_stage=1, inference_backend="native", synthetic_data=True,
                         synthetic_prompt_len=8, max_seq_len=16, max_data_samples=8, swift_sync_enabled=True,
                         swift_sync_fallback_full_every=3, warmup_steps=0, checkpoint_save_enabled=False,
                         output_dir=str(tmp_path), tensorboard=False, kv_num_blocks=32, amp_dtype="fp32")

    async def go():
        o = ColocateOrchestrator(cfg)
        await o.initialize()
        return o

    o = asyncio.run(go())
    eng = o.train_engine
    o.swift.worker.lowrank_on_cpu = True
    mods = [m for m in eng.model.modules() if isinstance(m, LinearWithLoRA)]
    assert any(len(m.adapters) > 1 for m in mods)             # fused q|k|v / gate|up: several adapters per module
    base0 = [m.base.weight.detach().clone() for m in mods]
    g = torch.Generator().manual_seed(3)
    modes = []
    for it in range(5):
        with torch.no_grad():
            for m in mods:
                for ad in m.adapters.values():
                    ad.lora_A.add_(0.05 * torch.randn(ad.lora_A.shape, generator=g))
                    ad.lora_B.add_(0.05 * torch.randn(ad.lora_B.shape, generator=g))
        o._sync_weights(it)
        modes.append(o.swift.stats.last_mode)
        got, want = dict(hf_named_tensors(o.infer_engine.model)), eng.export_weights()
        for k, v in want.items():
            assert torch.allclose(got[k].float(), v.float(), atol=2e-4, rtol=1e-4), (it, modes, k)
    assert "delta" in modes and "full" in modes
    assert o.swift.worker._plan is not None
    for m, w0 in zip(mods, base0):
        assert torch.equal(m.base.weight, w0)


def test_flat_adapter_state_takes_the_same_path_as_a_dict_of_tensors():
    """``FlatState`` (all adapter tensors in one flat tensor) through the delta computer, the double buffer and the
    transfer's commit gives what a plain dict of tensors gives; mixing the two falls back to the per-key path."""
    from b200fw.sync import DeltaComputer, DoubleBufferedLoRA, SwiftSyncConfig, SwiftSyncTransfer
    from b200fw.sync.double_buffer import FlatLayout, FlatState
    torch.manual_seed(0)
    shapes = {"a.lora_A": (4, 6), "a.lora_B": (10, 4), "b.lora_A": (4, 3)}
    layout = FlatLayout(list(shapes), list(shapes.values()))

    def state(seed):
        g = torch.Generator().manual_seed(seed)
        return FlatState(layout, torch.randn(layout.numel, generator=g))

    s0, s1, s2 = state(0), state(1), state(2)
    assert list(s0) == list(shapes) and "a.lora_B" in s0 and "zzz" not in s0 and s0["a.lora_B"].shape == (10, 4)
    assert s0["b.lora_A"].data_ptr() == s0.flat[64:].data_ptr()                   # a view, not a copy
    flat_dc, dict_dc = DeltaComputer(100), DeltaComputer(100)
    for cur in (s0, s1, s2):
        d_flat = flat_dc.compute_delta(FlatState(layout, cur.flat.clone()))
        d_dict = dict_dc.compute_delta({k: v.clone() for k, v in cur.items()})
        assert isinstance(d_flat, FlatState)
        for k in shapes:
            assert torch.equal(d_flat[k], d_dict[k])

    class Worker:
        def __init__(self):
            self.calls = []

        def update_weights(self, st, mode="full"):
            self.calls.append((mode, {k: v.clone() for k, v in st.items()}))

    wf, wd = Worker(), Worker()
    tf = SwiftSyncTransfer(wf, SwiftSyncConfig(True, fallback_full_every=100))
    td = SwiftSyncTransfer(wd, SwiftSyncConfig(True, fallback_full_every=100))
    for step, cur in enumerate((s0, s1, s2)):
        tf.sync(step, FlatState(layout, cur.flat.clone()))
        td.sync(step, {k: v.clone() for k, v in cur.items()})
    assert [m for m, _ in wf.calls] == [m for m, _ in wd.calls] == ["full", "delta", "delta"]
    for (_, a), (_, b) in zip(wf.calls, wd.calls):
        assert all(torch.equal(a[k], b[k]) for k in shapes)
    assert tf.buffer.version == td.buffer.version == 3
    fa, da = tf.buffer.get_active_state(), td.buffer.get_active_state()
    assert all(torch.allclose(fa[k], da[k], atol=1e-6) and torch.allclose(fa[k], s2[k], atol=1e-5) for k in shapes)
    assert tf.stats.last_bytes == td.stats.last_bytes == layout.numel * 4
    # a plain-dict delta on a flat buffer: the per-key path takes over and still lands in the same tensors
    buf = DoubleBufferedLoRA(s0)
    buf.apply_delta_to_shadow({"a.lora_A": torch.ones(4, 6), "new.lora_A": torch.ones(2, 2)})
    buf.swap_buffers()
    act = buf.get_active_state()
    assert torch.allclose(act["a.lora_A"], s0["a.lora_A"] + 1) and torch.equal(act["new.lora_A"], torch.ones(2, 2))


def test_resume_continues_the_loop_and_the_data_stream_where_the_checkpoint_left_them():
    """An SFT run interrupted after 2 of 4 iterations and resumed from ``iter_2`` produces, in iterations 2 and 3, the
    losses of the run that was never interrupted: the loop index, the data position, the weights, the optimizer
    moments and the learning-rate schedule all come back.  A checkpoint without the orchestrator's state file restores
    the engine only."""
    with tempfile.TemporaryDirectory() as d:
        common = dict(training_mode="sft", total_iterations=4, max_tokens=6, batch_size=2, inference_preview_enabled=False,
                      lr_scheduler_type="cosine", learning_rate=2e-3)
        whole, _ = _run(_tiny_cfg(os.path.join(d, "a"), checkpoint_save_enabled=False, **common))
        want = [m.train_metrics.loss for m in whole.metrics]
        assert len(want) == 4 and len(set(want)) == 4
        # the interrupted run: same schedule (total 4), stopped after iteration 2 by its checkpoint interval
        first_cfg = _tiny_cfg(os.path.join(d, "b"), checkpoint_save_interval=2, **common)
        first = ColocateOrchestrator(first_cfg)

        async def two_then_stop():
            await first.initialize()
            real = first._save_checkpoint

            def stop_after(tag, done=None):
                real(tag, done)
                if tag == "iter_2":
                    raise KeyboardInterrupt           # the process dies right after the checkpoint
            first._save_checkpoint = stop_after
            await first.run()
        with pytest.raises(KeyboardInterrupt):
            asyncio.run(two_then_stop())
        ck = os.path.join(first_cfg.checkpoint_save_dir, "iter_2")
        st = json.load(open(os.path.join(ck, "orchestrator_state.json")))
        assert st["iterations_completed"] == 2
        resumed, _ = _run(_tiny_cfg(os.path.join(d, "c"), resume_from=ck, checkpoint_save_enabled=False, **common))
        assert resumed.start_iteration == 2 and [m.iteration for m in resumed.metrics] == [2, 3]
        got = [m.train_metrics.loss for m in resumed.metrics]
        assert got == pytest.approx(want[2:], rel=1e-6), (got, want)
        # without the state file: engine restored, loop from 0
        os.remove(os.path.join(ck, "orchestrator_state.json"))
        plain, _ = _run(_tiny_cfg(os.path.join(d, "e"), resume_from=ck, checkpoint_save_enabled=False, **common))
        assert plain.start_iteration == 0 and len(plain.metrics) == 4 and plain.train_engine.step_count > 4


def test_replacing_one_stage_leaves_the_native_default_stages_in_the_loop():
    """A subclass that replaces only the weight-sync coroutine gets the staged loop, in which the rollout and training
    stages are the native defaults (``_do_inference`` / ``_do_training``): the run is the plain loop's run, iteration
    for iteration, and the replaced stage is called once per iteration with the iteration number."""
    calls = []

    class Counting(ColocateOrchestrator):
        async def _do_weight_sync(self, iteration: int = 0):
            calls.append(iteration)
            await super()._do_weight_sync(iteration)

    async def go(cls, cfg):
        o = cls(cfg)
        await o.initialize()
        await o.run()
        await o.shutdown()
        return o
    with tempfile.TemporaryDirectory() as d:
        plain = asyncio.run(go(ColocateOrchestrator, _tiny_cfg(os.path.join(d, "a"), checkpoint_save_enabled=False)))
        staged = asyncio.run(go(Counting, _tiny_cfg(os.path.join(d, "b"), checkpoint_save_enabled=False)))
    assert calls == [0, 1, 2] and staged._stages_overridden() and not plain._stages_overridden()
    assert [m.error for m in staged.metrics] == [None] * 3
    assert [m.train_metrics.loss for m in staged.metrics] == pytest.approx([m.train_metrics.loss for m in plain.metrics], rel=1e-6)
    assert [m.tokens_generated for m in staged.metrics] == [m.tokens_generated for m in plain.metrics]
    assert staged.weights_version == plain.weights_version == 3
    # the other default stages, called directly
    async def direct():
        o = ColocateOrchestrator(_tiny_cfg(os.path.join(tempfile.mkdtemp(), "c"), checkpoint_save_enabled=False))
        await o.initialize()
        b = o._next_batch()
        one = await o._do_inference(b, num_samples=1)
        two = await o._do_inference_async(b)
        assert [len(g) for g in one] == [1, 1] and [len(g) for g in two] == [2, 2]
        assert o.config.num_samples_per_prompt == 2                  # put back after the one-sample call
        m = await o._do_sft_training(o._next_batch()) if o.config.training_mode == "sft" else None
        await o._do_weight_sync_async(0)
        assert o.weights_version == 1 and m is None
        await o.shutdown()
    asyncio.run(direct())


def test_resumed_grpo_run_draws_the_samples_of_the_uninterrupted_one():
    """GRPO with sampling (temperature 1): the checkpoint carries the rollout engine's sampling state, so iterations 2
    and 3 of a run resumed from ``iter_2`` generate the same tokens, see the same rewards and reach the same losses
    as the run that was never interrupted."""
    with tempfile.TemporaryDirectory() as d:
        common = dict(total_iterations=4, temperature=1.0, top_p=0.95, max_tokens=6, learning_rate=2e-3,
                      synthetic_reward_dense_weight=1.0)          # a reward that depends on every sampled token
        whole, _ = _run(_tiny_cfg(os.path.join(d, "a"), checkpoint_save_enabled=False, **common))
        first_cfg = _tiny_cfg(os.path.join(d, "b"), checkpoint_save_interval=2, **common)
        first = ColocateOrchestrator(first_cfg)

        async def two_then_stop():
            await first.initialize()
            real = first._save_checkpoint

            def stop_after(tag, done=None):
                real(tag, done)
                if tag == "iter_2":
                    raise KeyboardInterrupt
            first._save_checkpoint = stop_after
            await first.run()
        with pytest.raises(KeyboardInterrupt):
            asyncio.run(two_then_stop())
        ck = os.path.join(first_cfg.checkpoint_save_dir, "iter_2")
        assert os.path.exists(os.path.join(ck, "rollout_rng_rank0.pt"))
        resumed, _ = _run(_tiny_cfg(os.path.join(d, "c"), resume_from=ck, checkpoint_save_enabled=False, **common))
        assert [m.iteration for m in resumed.metrics] == [2, 3]
        for a, b in zip(whole.metrics[2:], resumed.metrics):
            assert a.tokens_generated == b.tokens_generated and a.avg_reward == pytest.approx(b.avg_reward, abs=1e-7)
            assert a.train_metrics.loss == pytest.approx(b.train_metrics.loss, rel=1e-5, abs=1e-7)
        assert len({m.avg_reward for m in whole.metrics}) > 1          # the rewards did vary: the comparison means something


def test_a_stop_request_ends_the_run_at_an_iteration_boundary_with_a_resumable_checkpoint():
    """``request_stop()`` (what the script's SIGTERM handler calls) during iteration 1: the loop finishes that
    iteration, saves ``iter_2``, skips the final checkpoint, and a run resumed from there completes iterations 2 and 3
    with the losses of a run that was never stopped."""
    with tempfile.TemporaryDirectory() as d:
        common = dict(training_mode="sft", total_iterations=4, max_tokens=6, batch_size=2, inference_preview_enabled=False,
                      learning_rate=2e-3)
        whole, _ = _run(_tiny_cfg(os.path.join(d, "a"), checkpoint_save_enabled=False, **common))
        cfg = _tiny_cfg(os.path.join(d, "b"), **common)
        o = ColocateOrchestrator(cfg)

        async def go():
            await o.initialize()
            real = o._train_sft

            def train(batch):
                if len(o.metrics) == 1:
                    o.request_stop()                  # arrives in the middle of iteration 1
                return real(batch)
            o._train_sft = train
            await o.run()
            await o.shutdown()
        asyncio.run(go())
        assert o.stopped_early and [m.iteration for m in o.metrics] == [0, 1] and o.state == OrchestratorState.DONE
        saved = set(os.listdir(cfg.checkpoint_save_dir))
        assert "iter_2" in saved and "final" not in saved
        assert os.path.exists(os.path.join(cfg.output_dir, "run_summary.json"))
        ck = os.path.join(cfg.checkpoint_save_dir, "iter_2")
        resumed, _ = _run(_tiny_cfg(os.path.join(d, "c"), resume_from=ck, checkpoint_save_enabled=False, **common))
        assert not resumed.stopped_early and [m.iteration for m in resumed.metrics] == [2, 3]
        assert [m.train_metrics.loss for m in resumed.metrics] == pytest.approx(
            [m.train_metrics.loss for m in whole.metrics[2:]], rel=1e-6)
        # a request during the last iteration changes nothing: the run is complete anyway
        last = ColocateOrchestrator(_tiny_cfg(os.path.join(d, "e"), **{**common, "total_iterations": 1}))

        async def one():
            await last.initialize()
            last.request_stop()
            await last.run()
            await last.shutdown()
        asyncio.run(one())
        assert not last.stopped_early and "final" in os.listdir(last.config.checkpoint_save_dir)


def _dp_stop_worker(rank, world, tmp):
    """Only rank 1 is asked to stop, in the middle of iteration 0."""
    cfg = _tiny_cfg(os.path.join(tmp, "shared"), dp_size=world, zero_stage=1, total_iterations=4, batch_size=4,
                    num_samples_per_prompt=2, output_dir=os.path.join(tmp, f"out{rank}"))
    o = ColocateOrchestrator(cfg)

    async def go():
        await o.initialize()
        if rank == 1:
            real = o._rewards

            def rewards(ro):
                o.request_stop()
                return real(ro)
            o._rewards = rewards
        await o.run()
        await o.shutdown()
    asyncio.run(go())
    ck = os.path.join(cfg.checkpoint_save_dir, "iter_1")
    return o.stopped_early, [m.iteration for m in o.metrics], sorted(os.listdir(ck))


def test_a_stop_request_on_one_rank_stops_every_rank_after_the_same_iteration():
    from _dist_util import run_ranks
    with tempfile.TemporaryDirectory() as d:
        res = run_ranks(_dp_stop_worker, 2, d, timeout=600)
    for stopped, its, files in res:
        assert stopped and its == [0]
        assert {"optimizer_state_rank0.pt", "optimizer_state_rank1.pt", "orchestrator_state.json", "trainer_state.json",
                "rollout_rng_rank0.pt", "rollout_rng_rank1.pt"} <= set(files), files


def test_checkpoint_retention_keeps_the_newest_iteration_directories():
    with tempfile.TemporaryDirectory() as d:
        cfg = _tiny_cfg(d, training_mode="sft", inference_preview_enabled=False, total_iterations=5,
                        checkpoint_save_interval=1, checkpoint_keep_last=2)
        os.makedirs(os.path.join(cfg.checkpoint_save_dir, "iter_notes"))          # not ours: left alone
        _run(cfg)
        assert sorted(os.listdir(cfg.checkpoint_save_dir)) == ["final", "iter_4", "iter_5", "iter_notes", "latest"]
        st = json.load(open(os.path.join(cfg.checkpoint_save_dir, "iter_5", "orchestrator_state.json")))
        assert st["iterations_completed"] == 5


def test_a_tokenizer_larger_than_the_model_vocabulary_is_refused_at_initialize():
    from b200fw.data.pipeline import GSM8KDataPipeline, SimpleTokenizer

    class Big(SimpleTokenizer):
        vocab_size = 10 ** 6

        def __len__(self):
            return self.vocab_size
    recs = [{"question": f"{i}+1?", "answer": f"#### {i + 1}"} for i in range(8)]
    with tempfile.TemporaryDirectory() as d:
        cfg = _tiny_cfg(d, synthetic_data=False, checkpoint_save_enabled=False)
        data = GSM8KDataPipeline(records=recs, prompt_template="plain", tokenizer=Big())

        async def go():
            o = ColocateOrchestrator(cfg, data=data)
            try:
                await o.initialize()
            finally:
                await o.shutdown()
        with pytest.raises(ValueError, match="tokenizer has 1000000 ids"):
            asyncio.run(go())
