"""ZeRO stage 0/1/2/3 against torch.optim.AdamW, rank consistency, the non-finite guard, the 3-D global
gradient norm, schedules and optimizer state round-trip (gloo, CPU, fp32)."""
import math

import torch

from _dist_util import run_ranks
from b200fw.model import ModelConfig, ParallelTransformerModel
from b200fw.optim import LRSchedule, ZeROOptimizer, build_optimizer

CFG = ModelConfig(vocab_size=256, hidden_size=32, num_layers=2, num_heads=2, num_kv_heads=2, head_dim=16,
                  intermediate_size=48, max_position_embeddings=128, tie_word_embeddings=True)


def _data(seed, n=4, s=12):
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(0, CFG.vocab_size, (n, s), generator=g)
    labels = ids.clone()
    labels[:, :3] = -100
    return ids, labels


def _zero_worker(rank, world, stage, steps, accum):
    from b200fw.dist.context import ParallelContext
    ctx = ParallelContext.init_distributed(dp_size=world, backend="gloo")
    m = ParallelTransformerModel(CFG, ctx)
    m.init_weights(7)
    ref = ParallelTransformerModel(CFG)
    ref.init_weights(7)
    opt = build_optimizer(m.parameters(), stage, lr=1e-2, weight_decay=0.1, ctx=ctx, bucket_mb=0.02)
    ropt = torch.optim.AdamW(ref.parameters(), lr=1e-2, weight_decay=0.1)
    assert opt.stage == stage and len(opt.buckets) > 1
    for step in range(steps):
        for a in range(accum):
            # reference sees every rank's micro-batch (mean over ranks and accumulation steps)
            for r in range(world):
                ids, labels = _data(100 * step + 10 * a + r)
                (ref.loss(ids, labels) / (world * accum)).backward()
            ids, labels = _data(100 * step + 10 * a + rank)
            opt.pre_forward()
            opt.begin_backward(sync=a == accum - 1)
            m.loss(ids, labels, loss_scale=1.0 / accum).backward()
            opt.post_backward()
        gn = opt.clip_grad_norm(0.5)
        rn = torch.nn.utils.clip_grad_norm_(ref.parameters(), 0.5)
        assert abs(float(gn) - float(rn)) / float(rn) < 1e-3
        opt.step()
        opt.zero_grad()
        ropt.step()
        ropt.zero_grad()
    with opt.eval_mode():
        err = max((a - b).abs().max().item() for a, b in zip(m.parameters(), ref.parameters()))
        flat = torch.cat([p.detach().reshape(-1) for p in m.parameters()])
    if stage >= 3:
        assert all(p.numel() == 0 for p in m.parameters())      # released between steps
    assert opt.master.numel() < sum(p.numel() for p in ref.parameters()) or world == 1 or stage == 0
    import hashlib
    return err, hashlib.sha256(flat.numpy().tobytes()).hexdigest()


def test_zero_stages_match_adamw_dp2():
    for stage in (0, 1, 2, 3):
        res = run_ranks(_zero_worker, 2, stage, 3, 2)
        assert max(r[0] for r in res) < 2e-5, f"stage {stage}"
        assert res[0][1] == res[1][1], f"stage {stage}: ranks diverged"


def _prefetch_worker(rank, world):
    """ZeRO-3 gather prefetch bookkeeping, with fake events standing in for the side stream's."""
    from b200fw.dist.context import ParallelContext
    ctx = ParallelContext.init_distributed(dp_size=world, backend="gloo")
    m = ParallelTransformerModel(CFG, ctx)
    m.init_weights(3)
    opt = build_optimizer(m.parameters(), 3, lr=1e-2, ctx=ctx, bucket_mb=0.02)
    assert not opt.attach_prefetch_hooks(m)            # CPU: no side stream, nothing to overlap
    opt.overlap = True
    assert opt.attach_prefetch_hooks(m) and len(opt._prefetch_hooks) == CFG.num_layers + 1
    waited = []

    class Stream:
        def wait_event(self, ev):
            waited.append(ev)

        def wait_stream(self, other):
            pass

    real = torch.cuda.current_stream
    torch.cuda.current_stream = lambda *a, **k: Stream()
    try:
        opt.pre_forward(lazy=True)                      # gloo gather, synchronous
        n = len(opt.buckets)
        index = {id(p): i for i, b in enumerate(opt.buckets) for p in b.params}
        emb = index[id(m.embed_tokens)]
        assert opt._prefetch_first == [emb] and opt._gather_order[0] == emb and sorted(opt._gather_order) == list(range(n))
        pos = {b: k for k, b in enumerate(opt._gather_order)}      # gathers are queued in the order layers run
        firsts = [min(pos[index[id(p)]] for p in layer.parameters()) for layer in m.layers]
        assert firsts == sorted(firsts) and firsts[0] > pos[emb]
        opt._gather_events.update({i: i for i in range(n)})
        opt.wait_gathered(opt._prefetch_first)
        assert waited == [emb]
        seen_at_layer = []
        hooks = [layer.register_forward_pre_hook(lambda mod, a: seen_at_layer.append(list(waited))) for layer in m.layers]
        ids, labels = _data(rank)
        opt.begin_backward(sync=True)
        m.loss(ids, labels).backward()
        for h in hooks:
            h.remove()
        # every layer's own buckets were waited for before it ran; later layers' buckets were not all forced early
        for li, layer in enumerate(m.layers):
            need = {index[id(p)] for p in layer.parameters()}
            assert need <= set(seen_at_layer[li]), (li, need, seen_at_layer[li])
        assert len(seen_at_layer[0]) < n
        assert sorted(waited) == list(range(n)) and not opt._gather_events     # the final norm's hook drained the rest
        opt._gather_events[0] = "late"
        opt.post_backward()                             # releases the parameters: pending gathers are waited for first
        assert waited[-1] == "late" and not opt._gather_events
    finally:
        torch.cuda.current_stream = real
    return True


def test_zero3_gather_prefetch_hooks():
    assert all(run_ranks(_prefetch_worker, 2))


def test_zero_local_mode_single_process():
    m = ParallelTransformerModel(CFG)
    m.init_weights(1)
    opt = ZeROOptimizer(m.parameters(), lr=1e-2, stage=3)
    assert opt.world == 1 and opt.stage == 1        # degenerate local mode
    ids, labels = _data(0)
    m.loss(ids, labels).backward()
    opt.post_backward()
    assert float(opt.clip_grad_norm(1.0)) > 0
    opt.step()
    opt.zero_grad()


def test_nonfinite_gradients_skip_the_update():
    m = ParallelTransformerModel(CFG)
    m.init_weights(1)
    opt = ZeROOptimizer(m.parameters(), lr=1e-2, stage=1)
    before = [p.detach().clone() for p in m.parameters()]
    ids, labels = _data(0)
    m.loss(ids, labels).backward()
    next(m.parameters()).grad[0, 0] = float("nan")
    opt.post_backward()
    assert float(opt.clip_grad_norm(1.0)) == -1.0
    opt.step()
    assert all(torch.equal(a, b) for a, b in zip(before, m.parameters()))


def _norm_worker(rank, world, tp, pp, dp):
    """Global norm over a (pp, tp, dp) world equals the norm of the reassembled full gradient."""
    import torch.distributed as dist
    from b200fw.dist.context import ParallelContext
    ctx = ParallelContext.init_distributed(tp_size=tp, dp_size=dp, pp_size=pp, backend="gloo")
    g = torch.Generator().manual_seed(1000 + ctx.pp_rank * 10 + ctx.tp_rank)
    sharded = torch.nn.Parameter(torch.zeros(6, 8))
    sharded.tp_sharded = tp > 1
    g2 = torch.Generator().manual_seed(2000 + ctx.pp_rank)
    repl = torch.nn.Parameter(torch.zeros(8))
    opt = ZeROOptimizer([sharded, repl], lr=1e-3, stage=1, ctx=ctx)
    # every DP rank contributes a different gradient; the optimizer averages them
    gs = torch.empty(6, 8).normal_(generator=g) * (1 + ctx.dp_rank)
    gr = torch.empty(8).normal_(generator=g2) * (1 + ctx.dp_rank)
    sharded.grad, repl.grad = gs.clone(), gr.clone()
    opt.post_backward()
    got = float(opt.clip_grad_norm(0.0))
    # oracle: average over DP, then count sharded params once per (pp,tp) and replicated once per pp
    mean_factor = sum(1 + d for d in range(dp)) / dp
    sq = torch.zeros(1)
    sq += (gs / (1 + ctx.dp_rank) * mean_factor).pow(2).sum() if ctx.dp_rank == 0 else 0
    if ctx.dp_rank == 0 and ctx.tp_rank == 0:
        sq += (gr / (1 + ctx.dp_rank) * mean_factor).pow(2).sum()
    dist.all_reduce(sq)
    want = math.sqrt(float(sq))
    assert abs(got - want) / want < 1e-5, (got, want)
    return True


def test_grad_norm_3d_tp2_dp2():
    assert all(run_ranks(_norm_worker, 4, 2, 1, 2))


def test_grad_norm_3d_pp2_tp2_dp2():
    assert all(run_ranks(_norm_worker, 8, 2, 2, 2, timeout=600))


def _plain_norm_worker(rank, world, tp, pp, dp):
    """``TrainEngine._clip_grad_norm`` on an object without a bucketed optimizer (gradients in ``p.grad``): the norm
    covers every rank of the (pp, tp, dp) world, gradients are scaled in place only above the limit."""
    import types
    import torch.distributed as dist
    from b200fw.dist.context import ParallelContext
    from b200fw.train import TrainEngine
    ctx = ParallelContext.init_distributed(tp_size=tp, dp_size=dp, pp_size=pp, backend="gloo")
    torch.manual_seed(7 + rank)
    model = torch.nn.Sequential(torch.nn.Linear(8, 16, bias=False), torch.nn.Linear(16, 4, bias=False))
    for p in model.parameters():
        p.grad = torch.randn_like(p) * (rank + 1)
    sq = torch.stack([p.grad.double().pow(2).sum() for p in model.parameters()]).sum()
    dist.all_reduce(sq)
    want = math.sqrt(float(sq))
    stub = types.SimpleNamespace(model=model, parallel_ctx=ctx, metrics_collector=None,
                                 config=types.SimpleNamespace(max_grad_norm=1e30))
    before = [p.grad.clone() for p in model.parameters()]
    got = TrainEngine._clip_grad_norm(stub)
    assert abs(got - want) / want < 1e-9 and all(torch.equal(a, p.grad) for a, p in zip(before, model.parameters()))
    stub.config.max_grad_norm = want / 4
    TrainEngine._clip_grad_norm(stub)
    assert all(torch.allclose(p.grad, a / 4, rtol=1e-5) for a, p in zip(before, model.parameters()))
    if rank == 1:                       # a non-finite gradient on ONE rank: every rank must report it (and none hang)
        model[0].weight.grad.fill_(float("nan"))
    assert TrainEngine._clip_grad_norm(stub) == -1.0
    return True


def test_plain_grad_norm_unit_covers_all_parallel_groups():
    assert all(run_ranks(_plain_norm_worker, 4, 2, 1, 2))


def test_lr_schedule_shapes():
    s = LRSchedule(1e-3, "cosine", warmup_steps=10, total_steps=110, min_lr_ratio=0.1)
    assert abs(s.lr_at(0) - 1e-5) < 1e-12 and abs(s.lr_at(10) - 1e-3) < 1e-12
    assert abs(s.lr_at(110) - 1e-4) < 1e-12 and abs(s.lr_at(60) - (1e-4 + 9e-4 * 0.5)) < 1e-9
    lin = LRSchedule(1e-3, "linear", 0, 100, 0.0)
    assert abs(lin.lr_at(50) - 5e-4) < 1e-12
    assert LRSchedule(1e-3, "constant", 0, 0).lr_at(1234) == 1e-3


def test_optimizer_state_roundtrip():
    m = ParallelTransformerModel(CFG)
    m.init_weights(1)
    opt = ZeROOptimizer(m.parameters(), lr=1e-2, stage=1)
    ids, labels = _data(0)
    m.loss(ids, labels).backward()
    opt.post_backward()
    opt.clip_grad_norm(1.0)
    opt.step()
    opt.zero_grad()
    sd = opt.state_dict()
    assert sd["type"] == "zero1" and sd["step_count"] == 1
    m2 = ParallelTransformerModel(CFG)
    m2.init_weights(99)
    opt2 = ZeROOptimizer(m2.parameters(), lr=1e-2, stage=1)
    assert opt2.load_state_dict(sd)
    for a, b in zip(m.parameters(), m2.parameters()):
        assert torch.equal(a, b)
    assert not opt2.load_state_dict({**sd, "world": 4})


def test_reference_keyword_names_and_layout_view():
    """``optimizer_class`` / ``parallel_context`` keywords, the flat-vector view of the layout and the one-rank
    case (no group, nothing sharded), as the reference's optimizer exposes them."""
    import pytest
    import torch
    from b200fw.dist.context import ParallelContext
    from b200fw.optim.zero import ZeROOptimizer
    lin = torch.nn.Linear(32, 32, bias=False)
    ctx = ParallelContext(tp_size=2, tp_group=None, dp_size=1, dp_group=None)
    opt = ZeROOptimizer(lin.parameters(), optimizer_class=torch.optim.AdamW, parallel_context=ctx, lr=1e-3, weight_decay=0.0)
    assert opt.group is None and opt.world_size == 1
    assert opt.shard_size == opt.padded_size == 1024 == ZeROOptimizer._pad_to_divisible(1024, 8)
    assert ZeROOptimizer._pad_to_divisible(1025, 8) == 1032
    with pytest.raises(ValueError):
        ZeROOptimizer(lin.parameters(), optimizer_class=torch.optim.SGD, lr=1e-3)
    assert ParallelContext.init_distributed(tp_size=1, dp_size=1, backend="gloo", init_single_process=True).world_size == 1
