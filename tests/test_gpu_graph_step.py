"""The CUDA-graph replay of a training micro-step gives the same losses and weights as eager execution."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _run(graph: bool, steps: int = 6, lora_rank: int = 0, fuse: bool = True):
    from b200fw.model import PRESETS
    from b200fw.model.lora import LinearWithLoRA
    from b200fw.train import TrainConfig, TrainEngine
    torch.manual_seed(0)
    cfg = TrainConfig(model_preset="tiny128", lora_rank=lora_rank, grpo_beta=0.0, gradient_accumulation_steps=2,
                      learning_rate=1e-3, warmup_steps=0, amp_dtype="bf16", zero_stage=1, max_seq_len=256,
                      cuda_graph_step=graph)
    eng = TrainEngine(cfg).initialize()
    for mod in eng.model.modules():
        if isinstance(mod, LinearWithLoRA):
            mod.fuse_into_base = fuse
    V = PRESETS["tiny128"].vocab_size
    losses = []
    for s in range(steps * 2):
        g = torch.Generator().manual_seed(s)
        ids = torch.randint(0, V, (4, 256), generator=g)
        labels = ids.clone()
        labels[:, :100 + 7 * (s % 3)] = -100                  # the supervised-row count changes between batches
        m = eng.sft_step_tensors(ids, labels)                 # host tensors: indices computed on the host
        losses.append(m.loss)
    w = torch.cat([p.detach().float().reshape(-1)[:1000] for p in eng.model.parameters() if p.requires_grad])
    used = len(eng._graphs)
    return losses, w.cpu(), used


def test_graphed_micro_step_matches_eager():
    eager_l, eager_w, used0 = _run(False)
    graph_l, graph_w, used1 = _run(True)
    assert used0 == 0 and used1 >= 1                          # the graph path really ran
    assert all(abs(a - b) < 2e-2 for a, b in zip(eager_l, graph_l)), (eager_l, graph_l)
    assert (eager_w - graph_w).abs().max() < 2e-2


def test_lora_training_fused_graphed_eager_and_unfused_agree():
    """LoRA adapters trained three ways: the rank-r update inside the base GEMMs with the micro-step replayed as a CUDA
    graph (adapter gradients written into the optimizer's bucket views by the op), the same launched kernel by kernel,
    and base projection + two adapter GEMMs with gradients arriving through autograd."""
    ref_l, ref_w, _ = _run(False, lora_rank=8, fuse=False)
    eager_l, eager_w, used0 = _run(False, lora_rank=8)
    graph_l, graph_w, used1 = _run(True, lora_rank=8)
    assert used0 == 0 and used1 >= 1
    assert ref_l[-1] < ref_l[0]                                                    # the adapters do learn
    for other_l, other_w in ((eager_l, eager_w), (graph_l, graph_w)):
        assert all(abs(a - b) < 3e-2 for a, b in zip(ref_l, other_l)), (ref_l, other_l)
        assert (ref_w - other_w).abs().max() < 3e-2
