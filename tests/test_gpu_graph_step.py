"""The CUDA-graph replay of a training micro-step gives the same losses and weights as eager execution."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _run(graph: bool, steps: int = 6):
    from b200fw.model import PRESETS
    from b200fw.train import TrainConfig, TrainEngine
    torch.manual_seed(0)
    cfg = TrainConfig(model_preset="tiny128", lora_rank=0, grpo_beta=0.0, gradient_accumulation_steps=2,
                      learning_rate=1e-3, warmup_steps=0, amp_dtype="bf16", zero_stage=1, max_seq_len=256,
                      cuda_graph_step=graph)
    eng = TrainEngine(cfg).initialize()
    V = PRESETS["tiny128"].vocab_size
    losses = []
    for s in range(steps * 2):
        g = torch.Generator().manual_seed(s)
        ids = torch.randint(0, V, (4, 256), generator=g)
        labels = ids.clone()
        labels[:, :100 + 7 * (s % 3)] = -100                  # the supervised-row count changes between batches
        m = eng.sft_step_tensors(ids, labels)                 # host tensors: indices computed on the host
        losses.append(m.loss)
    w = torch.cat([p.detach().float().reshape(-1)[:1000] for p in eng.model.parameters()])
    used = len(eng._graphs)
    return losses, w.cpu(), used


def test_graphed_micro_step_matches_eager():
    eager_l, eager_w, used0 = _run(False)
    graph_l, graph_w, used1 = _run(True)
    assert used0 == 0 and used1 >= 1                          # the graph path really ran
    assert all(abs(a - b) < 2e-2 for a, b in zip(eager_l, graph_l)), (eager_l, graph_l)
    assert (eager_w - graph_w).abs().max() < 2e-2
