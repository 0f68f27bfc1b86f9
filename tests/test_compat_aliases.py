"""``b200fw.compat``: code written against the reference's ``src.*`` package layout imports unchanged.

The table below lists every ``from src.<module> import <names>`` (and ``import src.<module>``) that occurs in the
reference's own package, scripts and tests; each must resolve through the aliases to an object of this package."""
import importlib
import subprocess
import sys
import textwrap

import pytest

REFERENCE_IMPORTS = {
    "src.data.data_pipeline": ["GRPOBatch", "GSM8KDataPipeline"],
    "src.distributed": ["ParallelContext", "ParallelTransformerModel", "ZeROOptimizer", "ZeROStage2Optimizer", "ZeROStage3Optimizer", "comm"],
    "src.distributed.comm": ["AsyncAllReduce", "all_gather", "all_gather_last_dim", "all_reduce", "all_reduce_async", "broadcast", "copy_to_parallel_region", "gather_from_parallel_region", "recv_backward", "recv_forward", "reduce_from_parallel_region", "reduce_scatter", "send_backward", "send_backward_recv_forward", "send_forward", "send_forward_recv_backward"],
    "src.distributed.lora": ["LinearWithLoRA", "LoRAColumnParallel", "LoRALayer", "LoRARowParallel", "apply_lora", "get_lora_state_dict", "merge_lora_weights"],
    "src.distributed.parallel_context": ["ParallelContext"],
    "src.distributed.pipeline_parallel": ["PipelineParallelContext", "split_layers_to_stages"],
    "src.distributed.pipeline_scheduler": ["PipelineScheduler", "default_loss_fn"],
    "src.distributed.stream_manager": ["StreamManager"],
    "src.distributed.tensor_parallel": ["ColumnParallelLinear", "ParallelAttention", "ParallelMLP", "ParallelTransformerLayer", "ParallelTransformerModel", "RMSNorm", "RowParallelLinear", "load_from_hf_checkpoint"],
    "src.distributed.zero_optim": ["ZeROOptimizer"],
    "src.distributed.zero_optim_v2": ["ZeROStage2Optimizer"],
    "src.distributed.zero_optim_v3": ["ZeROStage3Optimizer"],
    "src.engines.c3po_plus": ["C3POConfig", "C3POPlusScheduler"],
    "src.engines.icepop": ["IcePopConfig", "IcePopFilter"],
    "src.engines.infer_worker": ["get_infer_worker_class"],
    "src.engines.train_engine": ["TrainConfig", "TrainEngine", "TrainMetrics"],
    "src.engines.train_worker": ["get_train_worker_class"],
    "src.inference.attention": ["HAS_FLASH_ATTN", "PagedAttention", "PartitionedPagedAttention", "store_kv_cache"],
    "src.inference.context": ["InferenceContext", "get_context", "reset_context", "set_context"],
    "src.inference.cuda_graph": ["CUDAGraphRunner"],
    "src.inference.engine": ["InferenceConfig", "InferenceEngine"],
    "src.inference.kv_cache": ["Block", "BlockPool", "BlockTable", "HAS_FP8", "KVCacheManager", "_FP8_DTYPE"],
    "src.inference.model_runner": ["ModelRunner", "ModelRunnerConfig"],
    "src.inference.prefix_cache": ["CachedBlock", "PrefixCache"],
    "src.inference.radix_cache": ["RadixAttentionCache", "RadixNode"],
    "src.inference.scheduler": ["ContinuousBatchingScheduler", "Request", "RequestState", "SchedulerOutput"],
    "src.inference.speculative": ["SpeculativeConfig", "SpeculativeDecoder"],
    "src.kernels": ["flash_attention_triton"],
    "src.orchestrator.colocate_orchestrator": ["ColocateConfig", "ColocateOrchestrator", "IterationMetrics", "OrchestratorState"],
    "src.orchestrator.disagg_orchestrator": ["DisaggConfig", "DisaggOrchestrator"],
    "src.profiling.comm_profiler": ["CommProfiler", "CommRecord"],
    "src.profiling.compute_profiler": ["ComputeProfiler", "LayerProfile"],
    "src.profiling.schedule_visualizer": ["ScheduleEvent", "ScheduleVisualizer"],
    "src.reward.gsm8k_reward": ["GSM8KRewardFunction", "compute_batch_rewards", "compute_reward"],
    "src.transfer.ipc_transfer": ["IPCHandle", "IPCWeightTransfer", "NON_RETRIABLE_EXCEPTIONS", "RETRIABLE_EXCEPTIONS", "TransferStats", "VLLMClient", "WeightUpdateManager"],
    "src.transfer.nccl_transfer": ["NCCLWeightTransfer", "RayObjectStoreTransfer", "WeightTransferManager"],
    "src.transfer.swift_sync": ["DeltaComputer", "DeltaVersion", "DoubleBufferedLoRA", "SwiftSyncConfig", "SwiftSyncTransfer"],
    "src.utils.artifact_writer": ["ArtifactWriter"],
    "src.utils.eval_utils": ["EvalMetrics", "compute_bleu4", "compute_exact_match", "compute_token_f1", "normalize_text"],
    "src.utils.logger": ["get_logger", "setup_logger"],
    "src.utils.memory_manager": ["MemoryManager"],
    "src.utils.memory_profiler": ["MemoryBreakdown", "MemoryProfiler", "MemoryReport", "MemorySnapshot"],
    "src.utils.metrics": ["MetricsCollector"],
}


@pytest.fixture()
def aliases():
    import b200fw.compat as compat
    had = compat.installed()
    if not compat.install():
        pytest.skip("a real `src` package is importable in this environment")
    yield compat
    if not had:
        compat.uninstall()


@pytest.mark.parametrize("module", sorted(REFERENCE_IMPORTS))
def test_every_name_the_reference_imports_resolves(aliases, module):
    m = importlib.import_module(module)
    missing = [n for n in REFERENCE_IMPORTS[module] if not hasattr(m, n)]
    assert not missing, (module, missing)
    assert all(t.startswith("b200fw") for t in m.__b200fw_targets__)


def test_aliases_give_the_same_objects_and_can_be_removed(aliases):
    from src.engines.train_engine import TrainConfig, TrainEngine
    from src.transfer.swift_sync import DoubleBufferedLoRA, SwiftSyncTransfer
    import b200fw.sync as sync
    import b200fw.train as train
    assert TrainEngine is train.TrainEngine and TrainConfig is train.TrainConfig
    assert DoubleBufferedLoRA is sync.DoubleBufferedLoRA and SwiftSyncTransfer is sync.SwiftSyncTransfer
    import src.kernels
    assert src.kernels.flash_attention_triton is None
    aliases.uninstall()
    assert not any(k == "src" or k.startswith("src.") for k in sys.modules)
    with pytest.raises(ImportError):
        importlib.import_module("src.engines.train_engine")
    assert aliases.install()


def test_reference_style_program_runs_through_the_aliases(tmp_path):
    """A small program in the reference's style (its imports, its constructor forms) in a fresh interpreter."""
    prog = tmp_path / "user_code.py"
    prog.write_text(textwrap.dedent("""
        import b200fw.compat
        assert b200fw.compat.install()
        import torch
        from src.distributed.parallel_context import ParallelContext
        from src.distributed.tensor_parallel import ParallelTransformerModel
        from src.distributed.lora import apply_lora
        from src.engines.icepop import IcePopConfig, IcePopFilter
        from src.inference.engine import InferenceConfig, InferenceEngine
        from src.transfer.swift_sync import DeltaComputer
        ctx = ParallelContext(tp_size=1, tp_group=None)
        model = ParallelTransformerModel(vocab_size=64, hidden_size=32, num_layers=2, num_heads=4, num_kv_heads=2,
                                         head_dim=8, intermediate_size=48, parallel_context=ctx,
                                         max_position_embeddings=32)
        logits = model(torch.randint(0, 64, (2, 8)))
        assert logits.shape == (2, 8, 64)
        names = apply_lora(model, rank=4, alpha=8.0)
        assert len(names) == 2 * 7
        eng = InferenceEngine(InferenceConfig(inference_mode="mock", vocab_size=64)).initialize()
        out = eng.generate([[5, 6, 7]], max_tokens=4)
        assert len(out[0]) == 4
        d = DeltaComputer(10)
        d.compute_delta({"a": torch.ones(2)})
        assert torch.equal(d.compute_delta({"a": torch.full((2,), 3.0)})["a"], torch.full((2,), 2.0))
        print("ok")
    """))
    import os
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, PYTHONPATH=root)
    r = subprocess.run([sys.executable, str(prog)], cwd=str(tmp_path), env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and r.stdout.strip().endswith("ok"), r.stderr[-2000:]


def test_reference_call_forms_of_module_level_functions(tmp_path):
    """Positional forms that differ from this package's own: ``apply_lora(model, dict, ctx)``,
    ``load_from_hf_checkpoint(model, path, ctx)``, ``set_context(is_prefill, cu_q, cu_k, ...)``,
    ``setup_logger(name, level, file, use_color)``, ``MemoryReport(model, optimizer, config)`` as a reporter object."""
    import torch
    from b200fw.dist.context import ParallelContext
    from b200fw.infer.context import get_context, reset_context, set_context
    from b200fw.model import ModelConfig, ParallelTransformerModel, apply_lora, load_from_hf_checkpoint, save_hf_checkpoint
    from b200fw.obs.logging import setup_logger
    from b200fw.obs.memory import MemoryReport, StepMemoryReporter
    ctx = ParallelContext(tp_size=1, tp_group=None)
    mc = ModelConfig(vocab_size=64, hidden_size=32, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=8,
                     intermediate_size=48, max_position_embeddings=32, tie_word_embeddings=False)
    src = ParallelTransformerModel(mc)
    src.init_weights(3)
    save_hf_checkpoint(src, str(tmp_path / "ckpt"))
    model = ParallelTransformerModel(mc)
    loaded, missing = load_from_hf_checkpoint(model, str(tmp_path / "ckpt"), ctx)
    assert loaded > 0 and missing == 0 and torch.equal(model.embed_tokens, src.embed_tokens)
    out = apply_lora(model, {"rank": 4, "alpha": 8.0, "target_modules": ["q_proj", "v_proj"], "dropout": 0.0}, ctx)
    assert out is model and len(model.lora_adapted_names) == 2 * 2
    assert all(("lora_" in n) == p.requires_grad for n, p in model.named_parameters())
    with pytest.raises(ValueError):
        apply_lora(ParallelTransformerModel(mc), {"rank": 4, "dropout": 0.1}, ctx)
    cu = torch.tensor([0, 3], dtype=torch.int32)
    c = set_context(True, cu, cu, 3, 3, torch.tensor([0, 1, 2]))
    assert c.is_prefill and c.max_seqlen_q == 3 and c.max_seqlen_k == 3 and get_context() is c and c.slot_mapping.numel() == 3
    reset_context()
    lg = setup_logger("b200fw.test_compat", "INFO", None, False)
    assert lg.handlers
    opt = torch.optim.AdamW([p for p in model.parameters() if p.requires_grad], lr=1e-3)
    rep = MemoryReport(model, opt, {"batch_size": 2})
    assert isinstance(rep, StepMemoryReporter)
    ids = torch.randint(0, 64, (2, 8))
    labels = ids.clone()
    labels[:, :4] = -100
    r = rep.profile_step(ids, labels, train_step_fn=None)
    assert set(r) >= {"model_spec", "static_memory", "dynamic_memory", "framework_overhead", "peak_moments"}
    assert r["model_spec"]["trainable_params"] == sum(p.numel() for p in model.parameters() if p.requires_grad)
    assert r["static_memory"]["optimizer_states_gb"] > 0 and "backward_peak_gb" in r["peak_moments"]
    assert rep.generate_report_without_step()["static_memory"]["static_total_gb"] > 0
    assert isinstance(MemoryReport(), MemoryReport)                     # the dataclass form is untouched


# keyword arguments the reference's entry scripts pass to the config classes (scripts/run_colocate.py,
# run_disaggregated.py, run_inference.py)
SCRIPT_CONFIG_KEYWORDS = {
    "ColocateConfig": ['model_path', 'tp_size', 'pp_size', 'num_micro_batches', 'dp_size', 'max_seq_len', 'use_flash_attn',
                       'attention_backend', 'use_gradient_checkpoint', 'training_mode', 'output_dir', 'checkpoint_save_dir',
                       'checkpoint_save_interval', 'checkpoint_save_enabled', 'resume_from', 'total_iterations', 'batch_size',
                       'train_steps_per_iteration', 'gradient_accumulation_steps', 'inference_backend', 'vllm_url',
                       'num_samples_per_prompt', 'max_tokens', 'temperature', 'top_p', 'lora_rank', 'lora_alpha',
                       'lora_target_modules', 'learning_rate', 'weight_decay', 'max_grad_norm', 'amp_dtype', 'grpo_beta',
                       'grpo_clip_eps', 'lr_scheduler_type', 'warmup_steps', 'min_lr_ratio', 'max_data_samples',
                       'dataset_name', 'dataset_config', 'dataset_split', 'prompt_template', 'prompt_field', 'input_field',
                       'response_field', 'answer_field', 'eval_max_tokens', 'eval_num_prompts', 'enable_comm_overlap',
                       'zero_stage', 'inference_preview_enabled', 'enable_profiling', 'profile_interval', 'icepop_enabled',
                       'icepop_divergence_threshold', 'icepop_max_mask_ratio', 'c3po_plus_enabled', 'c3po_plus_token_budget',
                       'c3po_plus_target_batch_tokens', 'c3po_plus_packing_strategy', 'swift_sync_enabled',
                       'swift_sync_fallback_full_every', 'swift_sync_double_buffer', 'async_pipeline_enabled',
                       'async_pipeline_max_staleness', 'async_pipeline_queue_size'],
    "DisaggConfig": ['model_path', 'train_tp_size', 'infer_tp_size', 'total_iterations', 'batch_size',
                     'num_samples_per_prompt', 'weight_sync_backend', 'overlap_training_inference', 'lora_rank',
                     'learning_rate', 'max_tokens'],
    "InferenceConfig": ['model_path', 'inference_mode', 'num_layers', 'num_heads', 'num_kv_heads', 'head_dim', 'hidden_size',
                        'vocab_size', 'num_blocks', 'block_size', 'max_num_batched_tokens', 'max_num_sequences',
                        'enable_prefix_caching', 'enable_cuda_graph', 'enable_async_scheduling',
                        'enable_partitioned_attention', 'temperature', 'top_p'],
}


def test_config_classes_take_every_keyword_the_reference_scripts_pass():
    import dataclasses
    from b200fw.config import ColocateConfig
    from b200fw.infer import InferenceConfig
    from b200fw.orch import DisaggConfig
    for cls in (ColocateConfig, DisaggConfig, InferenceConfig):
        fields = {f.name for f in dataclasses.fields(cls)}
        missing = [k for k in SCRIPT_CONFIG_KEYWORDS[cls.__name__] if k not in fields]
        assert not missing, (cls.__name__, missing)


def test_text_data_run_in_the_reference_style(tmp_path):
    """What the reference's ``scripts/run_colocate.py`` does with a YAML that names an HF model directory and a local
    JSONL dataset: ``ColocateConfig`` from the reference's keywords, ``ColocateOrchestrator.initialize`` / ``run`` /
    ``get_summary`` / ``shutdown``, SFT and GRPO, text prompts through a tokenizer, the artefact files."""
    pytest.importorskip("transformers")
    pytest.importorskip("tokenizers")
    import asyncio
    import json
    from tokenizers import Tokenizer, models, pre_tokenizers
    from transformers import PreTrainedTokenizerFast
    from b200fw.config import ColocateConfig
    from b200fw.model import ModelConfig, ParallelTransformerModel, save_hf_checkpoint
    from b200fw.orch import ColocateOrchestrator
    vocab = {"<pad>": 0, "<unk>": 1, "</s>": 2}
    words = "what is plus the sum answer".split() + [str(i) for i in range(40)] + ["####", "?", "."]
    for w in words:
        vocab.setdefault(w, len(vocab))
    tok = Tokenizer(models.WordLevel(vocab, unk_token="<unk>"))
    tok.pre_tokenizer = pre_tokenizers.Whitespace()
    mdir = tmp_path / "model"
    mc = ModelConfig(vocab_size=64, hidden_size=32, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=8,
                     intermediate_size=48, max_position_embeddings=128, tie_word_embeddings=False)
    m = ParallelTransformerModel(mc)
    m.init_weights(0)
    save_hf_checkpoint(m, str(mdir))
    PreTrainedTokenizerFast(tokenizer_object=tok, pad_token="<pad>", unk_token="<unk>", eos_token="</s>").save_pretrained(str(mdir))
    rows = [{"question": f"what is {i} plus {i + 1} ?", "answer": f"the sum is {2 * i + 1} . #### {2 * i + 1}"} for i in range(12)]
    (tmp_path / "data.jsonl").write_text("\n".join(json.dumps(r) for r in rows))
    for mode in ("sft", "grpo"):
        cfg = ColocateConfig(model_path=str(mdir), tp_size=1, pp_size=1, dp_size=1, num_micro_batches=1, max_seq_len=64,
                             use_flash_attn=False, attention_backend="sdpa", training_mode=mode,
                             output_dir=str(tmp_path / f"out_{mode}"), checkpoint_save_enabled=False, total_iterations=2,
                             batch_size=2, gradient_accumulation_steps=1, inference_backend="custom",
                             num_samples_per_prompt=2, max_tokens=4, lora_rank=4, lora_alpha=8.0, amp_dtype="fp32",
                             grpo_beta=0.01, warmup_steps=0, max_data_samples=8, dataset_name=str(tmp_path / "data.jsonl"),
                             dataset_split="train", prompt_field="question", response_field="answer",
                             answer_field="answer", zero_stage=1, eval_num_prompts=0)

        async def go():
            o = ColocateOrchestrator(cfg)
            await o.initialize()
            await o.run()
            s = o.get_summary()
            await o.shutdown()
            return s

        s = asyncio.run(go())
        assert s["results"]["completed_iterations"] == 2 and s["results"]["failed_iterations"] == 0
        out = tmp_path / f"out_{mode}"
        for name in ("config_snapshot.json", "run_summary.json", "metrics_rank0.jsonl", "loss_curve.csv"):
            assert (out / name).exists(), name


def test_constructor_and_method_orders_of_the_reference():
    """Positional orders that differ between the two code bases are told apart by type or magnitude."""
    import torch
    from b200fw.model.lora import LoRALayer
    from b200fw.obs.memory import MemoryManager
    from b200fw.obs.profilers import ComputeProfiler
    from b200fw.sync.nccl_transfer import NCCLWeightTransfer
    p = ComputeProfiler(device_name="B200", peak_tflops=1000.0)
    own = [p.compute_mfu(8e15, 1.0, 8), p.compute_mfu(flops=8e15, step_s=1.0, n_gpus=8), p.compute_mfu(8e15, step_s=1.0, n_gpus=8)]
    ref = [p.compute_mfu(1.0, 1e15), p.compute_mfu(actual_time_s=1.0, flops=1e15, device="B200", num_devices=8),
           p.compute_mfu(1.0, 1e15, "B200", 8)]
    assert all(abs(v - 1.0) < 1e-12 for v in own + ref) and p.compute_mfu(1e15, 0.0) == 0.0
    m = MemoryManager(0, 0.8, 0.9)
    assert (m.warn, m.critical, m.device) == (0.8, 0.9, torch.device("cuda", 0))
    m = MemoryManager(0.7, 0.9)
    assert (m.warn, m.critical, m.device) == (0.7, 0.9, None)
    m = MemoryManager(warning_threshold=0.6, critical_threshold=0.7)
    assert (m.warn, m.critical) == (0.6, 0.7) and MemoryManager().check() == "ok"
    t = NCCLWeightTransfer(1, "group")
    assert (t.group, t.src) == ("group", 1)
    t = NCCLWeightTransfer("group", 2)
    assert (t.group, t.src) == ("group", 2)
    t = NCCLWeightTransfer(src_rank=3, process_group="g")
    assert (t.group, t.src) == ("g", 3)
    assert LoRALayer(8, 8, 4, 8.0, 0.0).lora_A.shape == (4, 8)
    with pytest.raises(ValueError):
        LoRALayer(8, 8, 4, 8.0, 0.1)


def test_schedule_visualizer_in_both_call_forms():
    import time
    from b200fw.obs.timeline import ScheduleEvent, ScheduleVisualizer
    v = ScheduleVisualizer()
    v.add_event("F0", "forward", "stage0", 0.0, 5.0)                       # own form, milliseconds
    v.add_event("training", 0.010, 0.020, "GPU:1", tokens=5)                # the reference's form, seconds
    v.add_event("sync", 0.020, 0.021)
    with v.track("inference", "GPU:1", batch=3):
        time.sleep(0.001)
    with v.track("B0", "backward", "stage0"):
        pass
    with v.track("training"):
        pass
    e = {(x.name, x.lane): x for x in v.events}
    assert isinstance(v.events[0], ScheduleEvent)
    t = e[("training", "GPU:1")]
    assert (t.category, t.device, t.metadata) == ("backward", "GPU:1", {"tokens": 5})
    assert abs(t.start_time - 0.010) < 1e-12 and abs(t.duration_s - 0.010) < 1e-12 and abs(t.duration_ms - 10.0) < 1e-9
    assert e[("sync", "GPU:0")].category == "sync" and e[("inference", "GPU:1")].metadata == {"batch": 3}
    assert e[("B0", "stage0")].category == "backward" and ("training", "GPU:0") in e
    w = ScheduleVisualizer()
    w.add_event("F0", "forward", "stage0", 0.0, 10.0)
    assert v.compare(w)["speedup"] == ScheduleVisualizer.compare(v, w)["speedup"] > 0


def test_keyword_names_of_the_reference_on_transfer_metrics_and_cache_classes():
    import asyncio
    import torch
    from b200fw.infer import BlockPool
    from b200fw.obs.metrics import MetricsCollector
    from b200fw.obs.profilers import CommProfiler
    from b200fw.sync import DeltaComputer, IPCWeightTransfer, VLLMClient
    d = DeltaComputer(10)
    d.compute_delta(current_lora={"a": torch.ones(2)})
    assert torch.equal(d.compute_delta(current_lora={"a": torch.full((2,), 3.0)})["a"], torch.full((2,), 2.0))
    assert torch.equal(d.compute_delta(current_lora={"a": torch.ones(2)}, prev_lora={"a": torch.ones(2)})["a"], torch.zeros(2))
    with pytest.raises(TypeError):
        d.compute_delta(current={"a": torch.ones(2)}, current_lora={"a": torch.ones(2)})
    m = MetricsCollector()
    m.record(key="loss", value=2.0)
    assert m.series["loss"] == [2.0]
    ipc = IPCWeightTransfer(VLLMClient("http://127.0.0.1:9", timeout=1.0, max_retries=0, backoff_s=0.0))
    assert isinstance(ipc.build_ipc_handles(state_dict={"w": torch.ones(2)}), list)
    ipc.release_refs()
    pool = BlockPool(4, 16, 1, 1, 8, torch.float32, "cpu", cache_dtype="fp8")
    assert pool.fp8
    prof = CommProfiler()
    with prof.profile_op("all_reduce", torch.ones(1024), 2):
        pass
    with prof.profile_op(op_type="all_gather", tensor=torch.ones(8), world_size=2):
        pass
