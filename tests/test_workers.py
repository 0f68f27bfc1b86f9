"""TrainWorker / InferWorker: the reference's disaggregated worker API on top of the native engines (CPU)."""
import tempfile

import pytest
import torch

from b200fw.model import ModelConfig
from b200fw.model.hf_io import hf_named_tensors
from b200fw.orch import InferWorker, TrainWorker, get_infer_worker_class, get_train_worker_class
from b200fw.train import TrainConfig

SMALL = ModelConfig(vocab_size=256, hidden_size=32, num_layers=2, num_heads=2, num_kv_heads=2, head_dim=16,
                    intermediate_size=48, max_position_embeddings=256, tie_word_embeddings=False)


def _cfg(**kw):
    base = dict(model_config=SMALL, lora_rank=0, grpo_beta=0.0, learning_rate=1e-2, gradient_accumulation_steps=1,
                use_amp=False, amp_dtype="fp32", warmup_steps=0, max_seq_len=64)
    base.update(kw)
    return TrainConfig(**base)


def _rollout_data(seed=0, B=2, K=3):
    g = torch.Generator().manual_seed(seed)
    prompts = [torch.randint(3, 256, (6,), generator=g).tolist() for _ in range(B)]
    groups = [[torch.randint(3, 256, (4 + k,), generator=g).tolist() for k in range(K)] for _ in range(B)]
    rewards = [[1.0, 0.0, 0.5][:K], [0.1, 0.9, 0.3][:K]][:B]
    return prompts, groups, rewards


def test_train_worker_lifecycle_status_and_checkpoint():
    w = TrainWorker(_cfg())
    with pytest.raises(AssertionError):
        w.train_step(*_rollout_data())
    assert w.get_status()["initialized"] is False and "trainable_params" not in w.get_status()
    assert w.initialize() is True
    m = w.train_step(*_rollout_data())
    assert m.grad_norm > 0 and w.get_status()["step_count"] == 1
    st = w.get_status()
    assert st["trainable_params"] == st["total_params"] > 0 and st["total_train_time_s"] > 0
    assert st["config"] == {"model_path": w.config.model_path, "tp_size": 1, "lora_rank": 0}
    weights = w.export_weights()
    assert "model.embed_tokens.weight" in weights and "lm_head.weight" in weights
    with tempfile.TemporaryDirectory() as d:
        w.save_checkpoint(d)
        before = {k: v.clone() for k, v in w.export_weights().items()}
        w.sft_step([[5, 6, 7]], [[8, 9, 10, 11]])
        assert any(not torch.equal(before[k], v) for k, v in w.export_weights().items())
        assert w.load_checkpoint(d)
        assert all(torch.equal(before[k], v) for k, v in w.export_weights().items())
    assert get_train_worker_class() is TrainWorker and get_infer_worker_class() is InferWorker    # no Ray here


def test_infer_worker_mock_backend_and_errors():
    w = InferWorker()                                           # no model: scheduler + random tokens
    assert w.health_check() is False
    with pytest.raises(AssertionError):
        w.generate([[1, 2, 3]])
    w.initialize()
    assert w.health_check() and w.engine.config.inference_mode == "mock"
    out = w.generate([[5, 6, 7], [8, 9]], num_samples=3, max_tokens=5)
    assert len(out) == 2 and all(len(g) == 3 and all(1 <= len(o) <= 5 for o in g) for g in out)
    texts = w.generate(["hi there"], num_samples=2, max_tokens=4)      # byte tokenizer fallback: text in, text out
    assert len(texts) == 1 and len(texts[0]) == 2 and all(isinstance(t, str) for t in texts[0])
    assert w.update_weights({}, mode="full") and w.get_status()["weight_version"] == 1
    assert w.update_weights({}, mode="bogus") is False and w.get_status()["weight_version"] == 1
    st = w.get_status()
    assert st["total_requests"] == 3 and st["backend"] == "custom" and "scheduler" in st["engine_stats"]
    with pytest.raises(ValueError):
        InferWorker(backend="vllm")                      # the library backend needs a model directory
    with pytest.raises(ValueError):
        InferWorker(backend="nonsense")


def test_infer_worker_vllm_backend_drives_the_library_engine(monkeypatch):
    """``backend="vllm"`` builds ``vllm.LLM`` on the model directory and maps text / token-id prompts to its
    ``generate`` call, like the reference worker; checked against a stand-in module (no model files here)."""
    import sys
    import types
    calls = {}

    class FakeLLM:
        def __init__(self, **kw):
            calls["init"] = kw

        def generate(self, inputs, sp):
            calls["inputs"], calls["sp"] = inputs, sp
            comp = lambda i, k: types.SimpleNamespace(text=f"t{i}-{k}", token_ids=[i, k])
            return [types.SimpleNamespace(outputs=[comp(i, k) for k in range(sp.n)]) for i in range(len(inputs))]

    class FakeParams:
        def __init__(self, **kw):
            self.__dict__.update(kw)

    monkeypatch.setitem(sys.modules, "vllm", types.SimpleNamespace(LLM=FakeLLM, SamplingParams=FakeParams))
    w = InferWorker(model_path="/models/x", tp_size=2, backend="vllm", max_model_len=1024)
    assert w.initialize() and w.health_check()
    assert calls["init"]["model"] == "/models/x" and calls["init"]["tensor_parallel_size"] == 2
    out = w.generate(["hello", [4, 5, 6]], num_samples=2, max_tokens=7, temperature=0.5)
    assert out == [["t0-0", "t0-1"], [[1, 0], [1, 1]]]
    assert calls["inputs"][1] == {"prompt_token_ids": [4, 5, 6]} and calls["sp"].max_tokens == 7 and calls["sp"].top_p == 0.95
    assert w.update_weights({}, mode="full") is False and w.get_status()["backend"] == "vllm"


def test_trainer_to_rollout_weight_flow_full_and_delta():
    tw = TrainWorker(_cfg())
    tw.initialize()
    iw = InferWorker(model=tw.engine.model.clone(requires_grad=False))
    iw.initialize()
    assert iw.engine.config.inference_mode == "kv_cache"
    prompts = [[5, 6, 7, 8], [9, 10, 11]]
    a = iw.generate(prompts, num_samples=1, max_tokens=6, temperature=0.0)
    assert a == iw.generate(prompts, num_samples=1, max_tokens=6, temperature=0.0)          # greedy: repeatable
    for s in range(3):
        tw.train_step(*_rollout_data(s))
    assert iw.update_weights(tw.export_weights(), mode="full")
    mine = dict(hf_named_tensors(iw.engine.model))
    assert all(torch.equal(v, mine[k]) for k, v in tw.export_weights().items())
    assert iw.get_status()["weight_version"] == 1 and iw.engine.weights_version >= 1
    # delta mode: the first call seeds both buffers, later calls add to the shadow and swap
    merged = []

    def merge(active):
        merged.append({k: v.clone() for k, v in active.items()})
        return {}

    iw2 = InferWorker(model=tw.engine.model.clone(requires_grad=False), merge_fn=merge)
    iw2.initialize()
    assert iw2.update_weights({"a": torch.ones(2)}, mode="delta")
    assert iw2.update_weights({"a": torch.full((2,), 0.5)}, mode="delta")
    assert torch.equal(merged[-1]["a"], torch.full((2,), 1.5)) and iw2.get_status()["lora_buffer_version"] >= 1
    assert iw2.update_weights({"a": torch.ones(3)}, mode="delta") is False                  # wrong shape: rejected
    assert iw2.get_status()["weight_version"] == 2


def test_worker_classes_become_ray_actors_when_ray_is_importable(monkeypatch):
    """``get_train_worker_class`` / ``get_infer_worker_class`` wrap the plain classes with ``ray.remote(num_gpus=n)``
    when Ray imports (src/engines/train_worker.py:26-31, infer_worker.py:31-36); checked with a stand-in module."""
    import sys
    import types
    from b200fw.orch.workers import get_infer_worker_class, get_train_worker_class
    seen = []

    def remote(num_gpus=0):
        def wrap(cls):
            seen.append((cls.__name__, num_gpus))
            return types.SimpleNamespace(remote=lambda *a, **k: cls(*a, **k), cls=cls)
        return wrap

    monkeypatch.setitem(sys.modules, "ray", types.SimpleNamespace(remote=remote))
    tw, iw = get_train_worker_class(2), get_infer_worker_class(1)
    assert seen == [("TrainWorker", 2), ("InferWorker", 1)]
    w = iw.remote(backend="mock")
    assert w.initialize() and w.get_status()["backend"] == "mock"
    monkeypatch.delitem(sys.modules, "ray")
