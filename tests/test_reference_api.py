"""Public surface: classes keep the method, property and field names of the reference project, so that code written
against it finds them here.  The table lists names by class; a few of the adapters are exercised for behaviour."""
import importlib
import json

import pytest
import torch

SURFACE = {
    "b200fw.obs:ArtifactWriter": ["is_main", "write_main_json", "write_main_text", "write_rank_jsonl", "write_rank_json", "close"],
    "b200fw.obs:MetricsCollector": ["start_timer", "stop_timer", "record", "record_step", "get_summary", "to_tensorboard",
                                    "reset", "elapsed_time"],
    "b200fw.obs:CommProfiler": ["profile_op", "record_compute_time", "compute_bandwidth", "get_summary",
                                "get_theoretical_bandwidth", "report", "reset"],
    "b200fw.obs:ComputeProfiler": ["estimate_flops", "compute_mfu", "get_peak_tflops", "profile_layer", "profile_model",
                                   "report", "reset"],
    "b200fw.obs:ScheduleVisualizer": ["begin_event", "end_event", "track", "add_event", "render_ascii", "render_json",
                                      "get_utilization_stats", "compare", "report", "reset"],
    "b200fw.obs:MemoryProfiler": ["snapshot", "report", "get_timeline", "peak_memory_mb", "reset", "delta"],
    "b200fw.obs:MemoryBreakdown": ["analyze", "estimate", "report"],
    "b200fw.obs:MemoryReport": ["profile_step", "generate_report_without_step"],
    "b200fw.obs:MemoryManager": ["check_memory_pressure", "defragment", "reserve_buffer", "release_buffer", "get_stats"],
    "b200fw.obs:EvalMetrics": ["compute_single", "compute_batch", "get_summary", "reset"],
    "b200fw.dist.streams:StreamManager": ["compute_scope", "comm_scope", "transfer_scope", "sync_compute_to_comm",
                                          "sync_comm_to_compute", "sync_all", "get_stream_stats", "reset_stats"],
    "b200fw.dist.comm:AsyncAllReduce": ["start"],
    "b200fw.dist.comm:AsyncHandle": ["wait", "is_done"],
    "b200fw.dist.context:ParallelContext": ["rank", "prev_rank", "next_rank", "destroy"],
    "b200fw.pipeline.stages:PipelineParallelContext": ["pp_group", "stage_layer_range", "num_layers_this_stage",
                                                       "is_first_stage", "is_last_stage", "prev_rank", "next_rank"],
    "b200fw.pipeline.schedule_1f1b:PipelineScheduler": ["forward_step", "backward_step", "run_1f1b_schedule"],
    "b200fw.infer:Block": ["hash_value", "is_full", "reset"],
    "b200fw.infer:BlockPool": ["allocate", "free", "get_flattened_kv_cache", "num_free_blocks"],
    "b200fw.infer:CUDAGraphRunner": ["capture", "replay", "is_captured", "invalidate"],
    "b200fw.infer:ModelRunner": ["bind_kv_cache", "bind_hf_model", "run", "run_batch_decode", "prepare_prefill",
                                 "prepare_decode", "sample", "capture_cuda_graphs", "invalidate_cuda_graphs"],
    "b200fw.infer:SpeculativeDecoder": ["load_draft_model", "speculate", "verify", "sync_kv_cache", "acceptance_rate",
                                        "is_loaded", "get_stats"],
    "b200fw.infer:PagedAttention": ["forward"],
    "b200fw.infer:PartitionedPagedAttention": ["forward"],
    "b200fw.sync:TransferStats": ["start", "finish", "bandwidth_gbps", "total_time", "errors"],
    "b200fw.sync:NCCLWeightTransfer": ["broadcast_weights", "receive_weights", "current_version"],
    "b200fw.sync:RayObjectStoreTransfer": ["publish_weights", "fetch_weights", "has_new_version", "get_version_info",
                                           "current_version"],
    "b200fw.sync:WeightTransferManager": ["sync_weights", "sync_weights_sync", "current_version", "has_new_version",
                                          "get_transfer_stats"],
    "b200fw.sync:VLLMClient": ["health_check", "sleep", "wake_up", "reset_prefix_cache", "update_weights"],
    "b200fw.sync:IPCWeightTransfer": ["push_weights", "push_weights_sync", "verify_consistency", "release_refs"],
    "b200fw.sync:WeightUpdateManager": ["update_weights", "current_version", "rollback_count"],
    "b200fw.sync:DeltaComputer": ["compute_delta", "compute_delta_bytes", "should_full_sync"],
    "b200fw.sync:SwiftSyncTransfer": ["initialize", "sync_delta", "sync_full", "prev_snapshot", "double_buffer", "version",
                                      "initialized", "get_stats_summary"],
    "b200fw.sync:DoubleBufferedLoRA": ["apply_delta_to_shadow", "set_full_state", "swap_buffers", "get_active_state"],
    "b200fw.reward:GSM8KRewardFunction": ["accuracy", "format_accuracy", "average_reward", "reset_stats"],
    "b200fw.train:TrainEngine": ["trainable_params_count", "total_params_count", "sft_step", "grpo_step", "generate",
                                 "export_weights", "export_lora_delta", "save_checkpoint", "load_checkpoint"],
    "b200fw.optim:ZeROOptimizer": ["state_memory_usage", "total_optimizer_state_savings", "clip_grad_norm", "step", "zero_grad"],
    "b200fw.optim:ZeROStage3Optimizer": ["pre_forward", "post_backward", "pre_eval", "post_eval", "eval_mode"],
    "b200fw.orch:TrainWorker": ["initialize", "train_step", "export_weights", "get_status", "save_checkpoint", "load_checkpoint"],
    "b200fw.orch:InferWorker": ["initialize", "generate", "update_weights", "health_check", "get_status"],
}
RECORDS = ["b200fw.obs.profilers:CommRecord", "b200fw.obs.profilers:LayerProfile", "b200fw.obs.timeline:ScheduleEvent",
           "b200fw.obs.metrics:TimerRecord", "b200fw.sync:WeightVersion", "b200fw.sync:DeltaVersion", "b200fw.sync:SyncStats",
           "b200fw.sync:IPCHandle", "b200fw.infer:ModelRunnerConfig", "b200fw.infer:SpeculativeConfig"]


def _get(path):
    mod, name = path.split(":")
    return getattr(importlib.import_module(mod), name)


@pytest.mark.parametrize("path", sorted(SURFACE))
def test_class_keeps_the_reference_names(path):
    cls = _get(path)
    missing = [n for n in SURFACE[path] if not hasattr(cls, n)]
    assert not missing, f"{path}: {missing}"


def test_record_classes_exist():
    for path in RECORDS:
        assert isinstance(_get(path), type), path
    from b200fw.infer import get_context, reset_context, set_context, store_kv_cache      # noqa: F401
    from b200fw.dist.comm import all_reduce_async                                           # noqa: F401


SMALL = dict(vocab_size=64, hidden_size=32, num_layers=2, num_heads=2, num_kv_heads=1, head_dim=16, intermediate_size=48,
             max_position_embeddings=128, tie_word_embeddings=False)


def _model():
    from b200fw.model import ModelConfig, ParallelTransformerModel
    m = ParallelTransformerModel(ModelConfig(**SMALL))
    m.init_weights(0)
    return m.eval()


def test_observability_adapters(tmp_path):
    from b200fw.obs import ArtifactWriter, CommProfiler, ComputeProfiler, EvalMetrics, MemoryBreakdown, MemoryProfiler
    from b200fw.obs import MemoryReport, MetricsCollector, ScheduleVisualizer
    w = ArtifactWriter(str(tmp_path), 1, 2)
    w.write_rank_jsonl("metrics.jsonl", {"a": 1})
    w.write_rank_jsonl("metrics.jsonl", {"a": 2})
    ArtifactWriter(str(tmp_path), 1, 2).write_rank_jsonl("metrics.jsonl", {"a": 3})      # a new run truncates
    assert (tmp_path / "metrics_rank1.jsonl").read_text() == '{"a": 3}\n' and w.write_main_json("x.json", {}) is None
    m = MetricsCollector()
    m.record_step(grad_norm=1.5, learning_rate=1e-4)
    with m.timer("iteration"):
        pass
    s = m.get_summary()
    assert s["metrics"]["grad_norm"]["last"] == 1.5 and s["throughput"]["iterations_total"] == 1
    assert m.timer_records[0].name == "iteration" and m.timer_records[0].duration >= 0 and m.elapsed_time >= 0
    c = CommProfiler()
    c.add("all_reduce", 1 << 20, 8, 2.0)
    c.record_compute_time(8.0)
    assert abs(c.get_summary()["comm_ratio"] - 0.2) < 1e-9                               # comm / (comm + compute)
    assert abs(c.compute_bandwidth(1 << 30, 2.0, "all_reduce", 8) - 2 * 7 / 8 * (1 << 30) / 2e-3 / 1e9) < 1e-6
    assert c.compute_bandwidth(1 << 27, 1.0, "all_gather", 8) == pytest.approx(7 * (1 << 27) / 1e-3 / 1e9)
    assert c.get_theoretical_bandwidth() == 900.0 and "all_reduce" in c.report() and c.comm_records[0].world_size == 8
    c.reset()
    assert c.get_summary()["total_comm_ms"] == 0.0
    p = ComputeProfiler()
    f = p.estimate_flops(2, 128, 64, 2, 128, 1000, num_heads=4, head_dim=16)
    assert f["total"] == 3 * f["forward_total"] and f["forward_total"] == 2 * f["per_layer"] + f["lm_head"]
    assert p.get_peak_tflops("H20") == 148.0 and p.get_peak_tflops() == p.peak_tflops
    v = ScheduleVisualizer()
    v.begin_event("training", batch=4)
    v.end_event("training")
    v.end_event("never started")
    st = v.get_utilization_stats()
    assert list(st["stage_time_ms"]) == ["training"] and json.loads(v.render_json())["traceEvents"] and "GPU:0" in v.render_ascii()
    v.reset()
    assert v.render_ascii() == "(no events)"
    mp = MemoryProfiler()
    mp.snapshot("a")
    mp.snapshot("b")
    assert mp.delta("a", "b") == 0.0 and mp.delta("a", "missing") == 0.0 and mp.get_timeline()[0].stage == "a"
    lin = torch.nn.Linear(4, 4)

    def step(x, y):
        (lin(x) - y).pow(2).sum().backward()
    rep = MemoryReport.profile_step(torch.ones(2, 4), torch.zeros(2, 4), step, model=lin)
    assert "step" in rep.phase_peaks and lin.weight.grad is not None
    assert MemoryBreakdown.analyze(lin)["gradients_mb"] > 0 and "total" in MemoryBreakdown.estimate(10 ** 6).report()
    e = EvalMetrics()
    assert e.compute_batch(["a b c", "x"], ["a b c", "y"]) == {"token_f1": 0.5, "bleu4": 0.5, "exact_match": 0.5}
    assert e.get_summary()["token_f1_max"] == 1.0
    e.reset()
    assert e.get_summary() == {}


def test_runtime_adapters():
    from b200fw.dist.comm import AsyncAllReduce, all_reduce_async
    from b200fw.dist.streams import StreamManager
    from b200fw.pipeline.schedule_1f1b import PipelineScheduler
    from b200fw.pipeline.stages import PipelineParallelContext
    sm = StreamManager()
    a = AsyncAllReduce(None, sm)                       # the reference's (group, stream_manager) order
    assert a.group is None and a.sm is sm and AsyncAllReduce(sm).sm is sm
    h = a.start(torch.ones(2))
    assert h.is_done()
    h.wait()
    assert all_reduce_async(torch.ones(2), None, sm).is_done()
    with sm.comm_scope():
        pass
    assert sm.get_stream_stats()["comm_ops"] == 1
    sm.reset_stats()
    assert sm.get_stream_stats()["comm_ops"] == 0
    pp = PipelineParallelContext(5, pp_size=2, pp_rank=0)
    assert pp.stage_layer_range == (0, 3) and pp.num_layers_this_stage == 3 and pp.pp_group is None
    m = _model().train()
    sched = PipelineScheduler(m, PipelineParallelContext(2), 1)
    ids = torch.randint(0, 64, (2, 8))
    loss = sched.forward_step(m, ids, ids.clone())
    assert loss.dim() == 0 and sched.backward_step(None) is None and len(sched._fifo) == 0


def test_inference_adapters_match_the_native_path():
    from b200fw.infer import (InferenceConfig, InferenceEngine, ModelRunnerConfig, PagedAttention,
                              PartitionedPagedAttention, SpeculativeConfig, SpeculativeDecoder, reset_context, set_context,
                              store_kv_cache)
    from b200fw.model import ModelConfig
    m = _model()
    cfg = ModelConfig(**SMALL)
    eng = InferenceEngine(InferenceConfig.from_model_config(cfg, num_blocks=32, inference_mode="kv_cache"), m).initialize()
    r = eng.runner
    prompts = [[5, 6, 7, 8, 9], [10, 11, 12]]
    for i, p in enumerate(prompts):
        eng.kv.allocate_for_sequence(i, len(p))
    nxt = r.run(torch.tensor(prompts[0] + prompts[1]), r.prepare_prefill([0, 1], [0, 0], [5, 3])).argmax(-1)
    for i in range(2):
        eng.kv.append_token(i)
    ref = r.forward(nxt, r.prepare_decode([0, 1]))
    bt = torch.full((2, 4), -1, dtype=torch.int32)
    for i in range(2):
        t = eng.kv.get_block_table(i)
        bt[i, :len(t)] = torch.tensor(t)
    out = r.run_batch_decode(nxt[:, None], torch.tensor([5, 3]), bt, torch.tensor([6, 4]))
    assert torch.equal(out, ref)                                     # raw metadata tensors == manager-built context
    assert ModelRunnerConfig.from_runner(r).num_layers == 2 and r.capture_cuda_graphs() == []
    with pytest.raises(TypeError):
        r.bind_hf_model(torch.nn.Linear(2, 2))
    assert eng.pool.get_flattened_kv_cache().shape[2] == 32 * 16 and eng.pool.blocks[0].block_size == 16
    # module-style attention over a cache of its own
    from b200fw.infer import BlockPool
    Hq, Hkv, D, T = 2, 1, 16, 70
    pool = BlockPool(8, 16, 1, Hkv, D, torch.float32, torch.device("cpu"))
    kc, vc = pool.layer_kv(0)
    torch.manual_seed(0)
    K, V, blocks = torch.randn(T, Hkv, D), torch.randn(T, Hkv, D), [3, 1, 4, 0, 2]
    slots = torch.tensor([blocks[t // 16] * 16 + t % 16 for t in range(T)])
    slots[7] = -1                                                    # a skipped token leaves its slot untouched
    store_kv_cache(K, V, kc, vc, slots)
    assert torch.equal(kc[3, 0, 0], K[0, 0]) and torch.equal(vc[2, 5, 0], V[69, 0]) and float(kc[3, 7].abs().sum()) == 0.0
    kc[3, 7], vc[3, 7] = K[7], V[7]
    q = torch.randn(1, Hq, D)
    want = torch.softmax((q[0] @ K[:, 0].t()) * D ** -0.5, -1) @ V[:, 0]
    for cls, kw, split in ((PagedAttention, {}, (0, 1)), (PartitionedPagedAttention, {"partition_size": 64}, (64, 2))):
        att = cls(Hq, Hkv, D, **kw).bind_cache(kc, vc)
        ctx = set_context(False, num_seqs=1, block_tables=torch.tensor([blocks], dtype=torch.int32),
                          context_lens=torch.tensor([T], dtype=torch.int32), max_context_len=T)
        assert (att(q, K[-1:], V[-1:])[0] - want).abs().max() < 1e-5 and att._split(ctx) == split
    reset_context()
    with pytest.raises(RuntimeError):
        PagedAttention(Hq, Hkv, D)(q, K[-1:], V[-1:])
    # stateless speculate / verify: a draft identical to the target is accepted in full
    d = SpeculativeDecoder(None, m, config=SpeculativeConfig(enabled=True, num_speculative_tokens=3))
    ids = torch.randint(0, 64, (1, 5))
    dt, dl = d.speculate(ids)
    with torch.no_grad():
        tl = m(torch.cat([ids, dt[None]], 1))[:, -4:]
    acc, n = d.verify(ids, dt, tl)
    assert n == 3 and acc.tolist()[:3] == dt.tolist() and dl.shape == (3, 64)
    assert d.get_stats()["total_accepted"] == 3 and d.is_loaded and d.load_draft_model()


def test_transfer_adapters():
    from b200fw.orch import DisaggConfig
    from b200fw.orch.disagg import DisaggIterationMetrics
    from b200fw.sync import (DeltaComputer, IPCWeightTransfer, SwiftSyncConfig, SwiftSyncTransfer, TransferStats, VLLMClient,
                             WeightTransferManager, WeightUpdateManager, WeightVersion)

    class Eng:
        def load_weights(self, s):
            self.state = s
    mgr, eng = WeightTransferManager("local"), Eng()
    v = mgr.sync_weights_sync({"a": torch.ones(2)}, True, engine=eng)
    assert v.version == 1 and mgr.has_new_version(0) and not mgr.has_new_version(1) and "a" in eng.state
    assert mgr.get_transfer_stats()["total_syncs"] == 1 and WeightVersion().increment("x").checksum == "x"
    ts = TransferStats()
    ts.start()
    ts.finish()
    assert ts.total_time >= 0 and ts.bandwidth_gbps == 0.0 and ts.errors == 0
    t = SwiftSyncTransfer(None, SwiftSyncConfig(True, 10, True))
    assert not t.initialized
    t.initialize({"a": torch.ones(2)})
    assert t.initialized and t.sync(1, {"a": torch.full((2,), 1.5)}) == t.version
    s = t.get_stats_summary()
    assert s["total_delta_syncs"] == 1 and s["total_full_syncs"] == 0 and s["total_delta_bytes"] == 8
    assert torch.equal(t.double_buffer.get_active_state()["a"], torch.full((2,), 1.5)) and t.last_delta_version.delta_bytes == 8
    assert DeltaComputer.compute_delta_bytes({"a": torch.ones(3)}) == 12 and t.config.enable_double_buffer
    ipc = IPCWeightTransfer(VLLMClient("http://127.0.0.1:9", timeout=2.0, max_retries=0, backoff_s=0.0))
    st = {"w": torch.arange(4.0)}
    assert ipc.verify_consistency(st) and ipc.verify_consistency(st, ipc.checksum(st)) and not ipc.verify_consistency(st, "bad")
    assert ipc.push_weights_sync(st) is False                       # nothing listens there: reported, not raised
    ipc.release_refs()
    wm = WeightUpdateManager(torch.nn.Linear(1, 1))
    assert wm.current_version == 0 and wm.rollback_count == 0
    # the reference's keyword names and argument order on the transfer entry points
    assert wm.update_weights(new_state_dict={"weight": torch.full((1, 1), 3.0)}) and float(wm.model.weight) == 3.0
    mgr2, eng2 = WeightTransferManager("local"), Eng()
    mgr2.sync_weights({"b": torch.ones(1)}, is_sender=True, engine=eng2)
    mgr2.sync_weights(state_dict={"c": torch.ones(1)}, is_sender=True, engine=eng2)
    assert "c" in eng2.state and mgr2.version == 2
    t2 = SwiftSyncTransfer(None, SwiftSyncConfig(True, 10, True))
    assert t2.sync_full(full_state={"a": torch.ones(2)}) == 1
    c = DisaggConfig(num_train_gpus=2, num_infer_gpus=2)
    assert c.train_gpus == [0, 1] and c.infer_gpus == [2, 3] and c.infer_tp_size == 2 and c.overlap_training_inference
    assert DisaggIterationMetrics(0, rollout_time=1.5).infer_time == 1.5


def test_colocate_replaced_stages_drive_the_loop():
    """A caller (or subclass) that replaces ``_do_inference`` / ``_do_training`` / ``_do_weight_sync`` gets a loop that
    runs exactly those stages in order, with the sleep / wake calls of a server around the sync, and the collaborators
    are reachable under the reference's private names (tests/test_colocate_loop.py of the reference drives it so)."""
    import asyncio
    from b200fw.config import ColocateConfig
    from b200fw.data.pipeline import GRPOBatch
    from b200fw.orch.colocate import ColocateOrchestrator, OrchestratorState
    from b200fw.reward.gsm8k import GSM8KRewardFunction
    from b200fw.train.engine import TrainMetrics

    class Server:
        slept = woke = 0

        async def sleep(self, level=1):
            Server.slept += 1

        async def wake_up(self, tags=None):
            Server.woke += 1

    class Data:
        def get_batches(self, n):            # a list, not an iterator, and shorter than the run: it is cycled
            return [GRPOBatch(["6*7?"], [[5, 6, 7]], ["42"])]

    orch = ColocateOrchestrator(ColocateConfig(model_path="x", total_iterations=3, batch_size=1, num_samples_per_prompt=2,
                                               retry_delay=0.0))
    assert not orch._stages_overridden()
    orch._vllm_client, orch._reward_fn, orch._data_pipeline = Server(), GSM8KRewardFunction(), Data()
    assert orch.vllm_client is orch._vllm_client and orch.data is orch._data_pipeline
    order = []

    async def infer(batch):
        order.append("infer")
        return [["Step 1: 6*7=42\n#### 42", "Step 1: guess\n#### 41"] for _ in batch.prompts]

    async def train(batch, responses, rewards):
        order.append("train")
        assert rewards == [[1.0, -0.5]]
        if len(order) == 5:                  # second iteration fails in training
            raise RuntimeError("boom")
        return TrainMetrics(0.25, 0.2, 0.01, 1.0, 1e-5, step=len(order))

    async def sync():
        order.append("sync")

    orch._do_inference, orch._do_training, orch._do_weight_sync = infer, train, sync
    assert orch._stages_overridden()
    metrics = asyncio.run(orch.run())
    assert order == ["infer", "train", "sync", "infer", "train", "infer", "train", "sync"]
    assert len(metrics) == 3 and orch.state == OrchestratorState.DONE
    assert metrics[0].avg_reward == 0.25 and metrics[0].accuracy == 0.5 and metrics[0].train_metrics.loss == 0.25
    assert "boom" in metrics[1].error and metrics[2].error is None
    assert Server.slept == 2 and Server.woke == 3        # the failed iteration wakes the server on recovery
    assert set(metrics[0].state_durations) == {"inferring", "rewarding", "training", "syncing"}

    # the reference's (error, stage) call form of the recovery hook
    asyncio.run(orch._handle_error(RuntimeError("late"), "syncing"))
    assert orch.state == OrchestratorState.ERROR and Server.woke == 4


def _reference_form_pipeline_worker(rank, world):
    """The reference's way of building and driving a pipeline: the model from architecture keywords + ``pp_context``,
    ``PipelineScheduler(pp_context, num_micro_batches, loss_fn)``, ``run_1f1b_schedule(stage_model, iterator)``."""
    from b200fw.dist.context import ParallelContext
    from b200fw.model import ParallelTransformerModel
    from b200fw.pipeline import PipelineParallelContext, PipelineScheduler
    from b200fw.pipeline.schedule_1f1b import default_loss_fn
    arch = dict(vocab_size=64, hidden_size=32, num_layers=4, num_heads=4, num_kv_heads=2, head_dim=8,
                intermediate_size=48, max_position_embeddings=32)
    ctx = ParallelContext.init_distributed(tp_size=1, dp_size=1, pp_size=2, backend="gloo")
    ppc = PipelineParallelContext(ctx, num_layers=4)
    torch.manual_seed(5)
    full = ParallelTransformerModel(parallel_context=ParallelContext(tp_size=1, tp_group=None), **arch)
    g = torch.Generator().manual_seed(9)
    batches = [(torch.randint(0, 64, (2, 8), generator=g), torch.randint(0, 64, (2, 8), generator=g)) for _ in range(4)]
    ref = 0.0
    for ids, labels in batches:
        loss = default_loss_fn(full(ids), labels) / 4
        ref += float(loss)
        loss.backward()
    stage = ParallelTransformerModel(parallel_context=ctx, pp_context=ppc, use_gradient_checkpoint=False, **arch)
    assert stage.stage_start == ppc.stage_layer_range[0] and len(stage.layers) == 2
    assert (stage.embed_tokens is not None) == ppc.is_first_stage and (stage.norm is not None) == ppc.is_last_stage
    sd = full.state_dict()
    stage.load_state_dict({k: sd[k if not k.startswith("layers.") else
                                 f"layers.{int(k.split('.')[1]) + stage.stage_start}.{k.split('.', 2)[2]}"]
                           for k in stage.state_dict()})
    hidden_or_logits = stage(batches[0][0] if ppc.is_first_stage else torch.randn(2, 8, 32))
    assert hidden_or_logits.shape == ((2, 8, 32) if not ppc.is_last_stage else (2, 8, 64))
    stage.zero_grad(set_to_none=True)
    got = PipelineScheduler(ppc, num_micro_batches=4, loss_fn=default_loss_fn).run_1f1b_schedule(stage, iter(batches))
    if not ppc.is_last_stage:
        assert got is None
    else:
        assert abs(float(got) - ref) < 1e-5 * abs(ref)
    named = dict(full.named_parameters())
    for n, p in stage.named_parameters():
        k = n if not n.startswith("layers.") else f"layers.{int(n.split('.')[1]) + stage.stage_start}.{n.split('.', 2)[2]}"
        assert p.grad is not None and torch.allclose(p.grad, named[k].grad, atol=1e-5), n
    return True


def test_pipeline_in_the_reference_call_form_matches_the_full_model():
    from _dist_util import run_ranks
    assert all(run_ranks(_reference_form_pipeline_worker, 2))


def test_small_reference_named_helpers_compute_what_their_names_say():
    """Helpers that only exist because the reference's callers use them: a LoRA adapter called on its own, the ZeRO
    memory figures, re-binding a runner's KV pool, the transfer manager's version / statistics views and its coroutine
    form."""
    import asyncio
    from b200fw.infer import BlockPool, InferenceConfig, InferenceEngine, KVCacheManager
    from b200fw.model import ModelConfig, ParallelTransformerModel
    from b200fw.model.lora import LoRALayer
    from b200fw.optim import build_optimizer
    from b200fw.sync import WeightTransferManager
    torch.manual_seed(0)
    # ---- a LoRA adapter on its own: x A^T B^T * alpha / r ----
    ad = LoRALayer(16, 8, 4, 8.0)
    with torch.no_grad():
        ad.lora_B.normal_()
    x = torch.randn(5, 16)
    want = x @ ad.lora_A.t() @ ad.lora_B.t() * 2.0
    assert torch.allclose(ad(x), want, atol=1e-6) and torch.allclose(x @ ad.delta_weight().t(), want, atol=1e-5)
    with pytest.raises(ValueError):
        LoRALayer(16, 8, 4, 8.0, 0.1)                 # the reference's fifth positional argument: dropout
    # ---- ZeRO memory figures (one process: the whole state is local) ----
    lin = torch.nn.Linear(8, 8, bias=False)
    opt = build_optimizer(lin.parameters(), 1, lr=1e-3)
    assert opt.state_memory_usage == 2 * 4 * opt.exp_avg.numel()
    assert "Savings: 0.0%" in opt.total_optimizer_state_savings and "ZeRO-" in opt.total_optimizer_state_savings
    # ---- the runner can be pointed at another pool ----
    mc = ModelConfig(vocab_size=64, hidden_size=32, num_layers=2, num_heads=2, num_kv_heads=2, head_dim=16,
                     intermediate_size=48, max_position_embeddings=64, tie_word_embeddings=True)
    m = ParallelTransformerModel(mc)
    m.init_weights(0)
    eng = InferenceEngine(InferenceConfig.from_model_config(mc, num_blocks=8, inference_mode="kv_cache", temperature=0.0,
                                                            eos_token_id=None), m).initialize()
    first = eng.generate([[3, 4, 5, 6]], max_tokens=4)
    pool2 = BlockPool(8, 16, 2, 2, 16, torch.float32, "cpu")
    mgr2 = KVCacheManager(pool2, 16)
    eng.runner.bind_kv_cache(pool2, mgr2)
    eng.pool, eng.kv = pool2, mgr2
    assert eng.runner.pool is pool2 and eng.runner.mgr is mgr2
    assert eng.generate([[3, 4, 5, 6]], max_tokens=4) == first and pool2.num_free_blocks == 8
    assert eng.runner.capture_cuda_graphs([1, 2]) == []            # no graph runner on CPU
    eng.runner.invalidate_cuda_graphs()                             # and nothing to drop
    with pytest.raises(TypeError):
        eng.runner.bind_hf_model(torch.nn.Linear(2, 2))
    # ---- transfer manager views ----
    tm = WeightTransferManager()
    assert tm.get_version_info().version == int(tm.version) == tm.current_version.version
    st = tm.get_stats()
    assert {"backend", "version", "transfers", "total_bytes", "failures"} <= set(st)
    assert asyncio.iscoroutinefunction(tm.sync_weights_async)
