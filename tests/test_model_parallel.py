"""Tensor-parallel layers, sequence parallelism, LoRA x TP and HF shard IO against single-process
references (gloo, CPU, fp32)."""
import copy
import tempfile

import torch

from _dist_util import run_ranks
from b200fw.model import (PRESETS, ModelConfig, ParallelTransformerModel, apply_lora, get_lora_state_dict,
                          load_from_hf_checkpoint, merge_lora_weights, save_hf_checkpoint)

CFG = ModelConfig(vocab_size=512, hidden_size=64, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=16,
                  intermediate_size=96, max_position_embeddings=256, tie_word_embeddings=False)


def _full_model(path):
    torch.manual_seed(0)
    m = ParallelTransformerModel(CFG)
    m.init_weights(3)
    save_hf_checkpoint(m, path)
    return m


def _tp_worker(rank, world, path, seq_par):
    from b200fw.dist.context import ParallelContext
    ctx = ParallelContext.init_distributed(tp_size=world, backend="gloo")
    ref = ParallelTransformerModel(CFG)
    load_from_hf_checkpoint(ref, path, strict=True)
    m = ParallelTransformerModel(CFG, ctx, sequence_parallel=seq_par)
    loaded, missing = load_from_hf_checkpoint(m, path, strict=True)
    assert missing == 0
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, CFG.vocab_size, (2, 16), generator=g)
    labels = ids.clone()
    labels[:, :4] = -100
    out = m(ids)
    want = ref(ids)
    assert (out - want).abs().max() < 1e-4
    l, lr = m.loss(ids, labels), ref.loss(ids, labels)
    assert abs(l.item() - lr.item()) < 1e-5
    l.backward()
    lr.backward()
    # sharded weight grads equal the matching slice of the reference grads
    gw = m.layers[0].mlp.down_proj.weight.grad
    rw = ref.layers[0].mlp.down_proj.weight.grad
    n = rw.shape[1] // world
    assert (gw - rw[:, rank * n:(rank + 1) * n]).abs().max() < 1e-5, ((gw - rw[:, rank * n:(rank + 1) * n]).abs().max(), rw.abs().max())
    gq = m.layers[1].self_attn.qkv_proj.weight.grad
    rq = ref.layers[1].self_attn.qkv_proj.weight.grad
    D, hq, hk = CFG.head_dim, CFG.num_heads // world, CFG.num_kv_heads // world
    want_q = rq[rank * hq * D:(rank + 1) * hq * D]
    assert (gq[:hq * D] - want_q).abs().max() < 1e-5
    # partial-grad parameters need the TP sum; replicated ones are already complete
    import torch.distributed as dist
    qn = m.layers[0].self_attn.q_norm.weight
    assert qn.tp_partial_grad
    tot = qn.grad.clone()
    dist.all_reduce(tot, group=ctx.tp_group)
    assert (tot - ref.layers[0].self_attn.q_norm.weight.grad).abs().max() < 1e-5
    ln = m.layers[0].input_layernorm.weight
    if seq_par:
        assert ln.tp_partial_grad
        t2 = ln.grad.clone()
        dist.all_reduce(t2, group=ctx.tp_group)
        assert (t2 - ref.layers[0].input_layernorm.weight.grad).abs().max() < 1e-5
    else:
        assert not ln.tp_partial_grad
        assert (ln.grad - ref.layers[0].input_layernorm.weight.grad).abs().max() < 1e-5
    assert (m.embed_tokens.grad - ref.embed_tokens.grad).abs().max() < 1e-5
    # the untied LM head is sharded over the vocabulary; its grad is the matching row slice
    assert m.vocab_parallel and m.lm_head.shape[0] == CFG.vocab_size // world and m.lm_head.tp_sharded
    vl = CFG.vocab_size // world
    assert (m.lm_head.grad - ref.lm_head.grad[rank * vl:(rank + 1) * vl]).abs().max() < 1e-5
    lp, lpr = m.token_logprobs(ids, temperature=0.7), ref.token_logprobs(ids, temperature=0.7)
    assert (lp - lpr).abs().max() < 1e-4
    # gathered export equals the original full tensors
    from b200fw.model.hf_io import hf_named_tensors
    full = dict(hf_named_tensors(m))
    refd = dict(hf_named_tensors(ref))
    assert all((full[k] - refd[k]).abs().max() < 1e-7 for k in refd)
    return True


def test_tp2_matches_single():
    with tempfile.TemporaryDirectory() as d:
        _full_model(d)
        assert all(run_ranks(_tp_worker, 2, d, False))


def test_tp2_sequence_parallel_matches_single():
    with tempfile.TemporaryDirectory() as d:
        _full_model(d)
        assert all(run_ranks(_tp_worker, 2, d, True))


def test_hf_roundtrip_and_tied_presets():
    with tempfile.TemporaryDirectory() as d:
        m = _full_model(d)
        m2 = ParallelTransformerModel(CFG)
        loaded, missing = load_from_hf_checkpoint(m2, d, strict=True)
        assert missing == 0 and loaded > 0
        ids = torch.randint(0, CFG.vocab_size, (1, 8))
        assert torch.equal(m(ids), m2(ids))
    tiny = ParallelTransformerModel(PRESETS["tiny"])
    assert tiny.tied and tiny.lm_head is None
    assert sum(p.numel() for p in tiny.parameters()) == PRESETS["tiny"].num_params()
    assert PRESETS["qwen3-0.6b"].num_params() == 596049920


def test_gradient_checkpointing_same_grads():
    torch.manual_seed(0)
    a = ParallelTransformerModel(CFG)
    a.init_weights(1)
    b = copy.deepcopy(a)
    b.gradient_checkpointing = True
    ids = torch.randint(0, CFG.vocab_size, (2, 12))
    a.loss(ids, ids).backward()
    b.loss(ids, ids).backward()
    for pa, pb in zip(a.parameters(), b.parameters()):
        assert (pa.grad - pb.grad).abs().max() < 1e-6


def test_lora_single_process_merge_and_freeze():
    torch.manual_seed(0)
    m = ParallelTransformerModel(CFG)
    m.init_weights(2)
    ids = torch.randint(0, CFG.vocab_size, (2, 10))
    base = m(ids).detach()
    names = apply_lora(m, rank=4, alpha=8.0)
    assert len(names) == 7 * CFG.num_layers
    assert all(("lora_" in n) == p.requires_grad for n, p in m.named_parameters())
    assert torch.allclose(m(ids), base, atol=1e-6)          # B starts at zero
    for _, p in m.named_parameters():
        if p.requires_grad and p.shape[1] == 4:                # lora_B
            torch.nn.init.normal_(p, std=0.05)
    with_lora = m(ids).detach()
    assert (with_lora - base).abs().max() > 1e-4
    merge_lora_weights(m)
    assert torch.allclose(m(ids), with_lora, atol=1e-4)
    merge_lora_weights(m, unmerge=True)
    assert torch.allclose(m(ids), with_lora, atol=1e-4)
    assert len(get_lora_state_dict(m)) == 2 * 7 * CFG.num_layers


def _lora_tp_worker(rank, world, path):
    from b200fw.dist.context import ParallelContext
    ctx = ParallelContext.init_distributed(tp_size=world, backend="gloo")
    m = ParallelTransformerModel(CFG, ctx)
    load_from_hf_checkpoint(m, path, strict=True)
    apply_lora(m, rank=4, alpha=8.0)
    g = torch.Generator().manual_seed(5)
    for n, p in m.named_parameters():      # same replicated values on all ranks, distinct shards
        if "lora_" in n:
            with torch.no_grad():
                p.copy_(torch.empty(p.shape).normal_(0, 0.05, generator=g))
    ids = torch.randint(0, CFG.vocab_size, (2, 10), generator=torch.Generator().manual_seed(2))
    out = m(ids).detach()
    merge_lora_weights(m)
    merged = m(ids).detach()
    assert (out - merged).abs().max() < 1e-4
    return out.tolist()


def test_lora_tp2_merge_consistent_across_ranks():
    with tempfile.TemporaryDirectory() as d:
        _full_model(d)
        outs = run_ranks(_lora_tp_worker, 2, d)
        assert (torch.tensor(outs[0]) - torch.tensor(outs[1])).abs().max() < 1e-5


def _lora_sp_worker(rank, world, path):
    """LoRA x TP x sequence parallelism against the same adapters on an unsharded model: equal loss, and
    adapter gradients that match the unsharded ones (shards: the matching slice; partial-gradient
    tensors: after the sum over the TP group)."""
    import torch.distributed as dist
    from b200fw.dist.context import ParallelContext
    from b200fw.model.lora import iter_lora
    ctx = ParallelContext.init_distributed(tp_size=world, backend="gloo")
    ref = ParallelTransformerModel(CFG)
    load_from_hf_checkpoint(ref, path, strict=True)
    apply_lora(ref, rank=4, alpha=8.0)
    m = ParallelTransformerModel(CFG, ctx, sequence_parallel=True)
    load_from_hf_checkpoint(m, path, strict=True)
    apply_lora(m, rank=4, alpha=8.0)
    g = torch.Generator().manual_seed(5)
    full = {}
    for name, tgt, mod, ad in iter_lora(ref):
        with torch.no_grad():
            ad.lora_A.copy_(torch.empty(ad.lora_A.shape).normal_(0, 0.05, generator=g))
            ad.lora_B.copy_(torch.empty(ad.lora_B.shape).normal_(0, 0.05, generator=g))
        full[(name, tgt)] = ad
    for name, tgt, mod, ad in iter_lora(m):
        fa = full[(name, tgt)]
        with torch.no_grad():
            if ad.lora_A.shape == fa.lora_A.shape:
                ad.lora_A.copy_(fa.lora_A)
            else:                                              # row parallel: A sharded along its columns
                n = ad.lora_A.shape[1]
                ad.lora_A.copy_(fa.lora_A[:, rank * n:(rank + 1) * n])
            if ad.lora_B.shape == fa.lora_B.shape:
                ad.lora_B.copy_(fa.lora_B)
            else:                                              # column parallel: B sharded along its rows
                n = ad.lora_B.shape[0]
                ad.lora_B.copy_(_shard_rows_like(fa.lora_B, tgt, rank, world))
    ids = torch.randint(0, CFG.vocab_size, (2, 16), generator=torch.Generator().manual_seed(2))
    labels = ids.clone()
    labels[:, :5] = -100
    l, lr = m.loss(ids, labels), ref.loss(ids, labels)
    assert abs(l.item() - lr.item()) < 1e-5, (l.item(), lr.item())
    l.backward()
    lr.backward()
    worst = 0.0
    for name, tgt, mod, ad in iter_lora(m):
        fa = full[(name, tgt)]
        for leaf in ("lora_A", "lora_B"):
            p, fp = getattr(ad, leaf), getattr(fa, leaf)
            gr = p.grad.clone()
            if getattr(p, "tp_partial_grad", False):
                dist.all_reduce(gr, group=ctx.tp_group)
            if gr.shape == fp.grad.shape:
                want = fp.grad
            elif leaf == "lora_A":
                n = gr.shape[1]
                want = fp.grad[:, rank * n:(rank + 1) * n]
            else:
                want = _shard_rows_like(fp.grad, tgt, rank, world)
            worst = max(worst, float((gr - want).abs().max()))
    assert worst < 1e-5, worst
    return worst


def _shard_rows_like(t, tgt, rank, world):
    n = t.shape[0] // world
    return t[rank * n:(rank + 1) * n]


def test_lora_tp2_sequence_parallel_gradients_match_unsharded():
    with tempfile.TemporaryDirectory() as d:
        _full_model(d)
        run_ranks(_lora_sp_worker, 2, d)


def test_lora_linear_autograd_function_against_plain_autograd():
    """The fused LoRA linear's hand-written backward (run here through the GEMM op's CPU forms): gradients of x, the
    stacked adapters and the residual against autograd of the plain formula."""
    from b200fw.ops.gemm import _LoRALinear, gemm
    torch.manual_seed(1)
    M, K, N, R = 40, 24, 56, 16
    x, a, b, r = [torch.randn(*sh, requires_grad=True) for sh in ((M, K), (R, K), (N, R), (M, N))]
    w = torch.randn(N, K)
    y = _LoRALinear.apply(x, w, a, b, r, None)
    g = torch.randn(M, N)
    y.backward(g)
    x2, a2, b2, r2 = [t.detach().clone().requires_grad_() for t in (x, a, b, r)]
    y2 = x2 @ w.t() + (x2 @ a2.t()) @ b2.t() + r2
    y2.backward(g)
    assert torch.allclose(y, y2, atol=1e-4)
    for got, want in ((x.grad, x2.grad), (a.grad, a2.grad), (b.grad, b2.grad), (r.grad, r2.grad)):
        assert torch.allclose(got, want, atol=1e-4, rtol=1e-4)
    # the extended GEMM by itself, both layouts of the second operand
    A2, B2 = torch.randn(M, R), torch.randn(N, R)
    assert torch.allclose(gemm(x.detach(), w, ext=(A2, B2)), x.detach() @ w.t() + A2 @ B2.t(), atol=1e-4)
    assert torch.allclose(gemm(g, w, b_mn=True, ext=(A2, a.detach())), g @ w + A2 @ a.detach(), atol=1e-4)


def test_lora_linear_hands_stacked_gradients_to_the_adapters_parameters():
    """The plan form: stacked operands built without autograd, every adapter's fp32 A / B receives its slice of the
    stacked gradient (B's times the scaling), into ``main_grad`` when the parameter has one (overwrite, then
    accumulate) and through autograd otherwise."""
    from b200fw.ops.gemm import _LoRALinear
    torch.manual_seed(2)
    M, K, N = 24, 16, 40
    rows, ranks, scal = [(0, 16), (16, 24), (24, 40)], [8, 8, 8], [2.0, 0.5, 1.0]
    As = [torch.randn(r, K, requires_grad=True) for r in ranks]
    Bs = [torch.randn(e - s, r, requires_grad=True) for (s, e), r in zip(rows, ranks)]
    x = torch.randn(M, K, requires_grad=True)
    w, g = torch.randn(N, K), torch.randn(M, N)

    def stacked():
        a_cat = torch.cat(As, 0)
        b_bd = torch.zeros(N, sum(ranks))
        r0 = 0
        for B, (s0, e0), r, sc in zip(Bs, rows, ranks, scal):
            b_bd[s0:e0, r0:r0 + r] = B * sc
            r0 += r
        return a_cat, b_bd

    y_ref = x @ w.t() + (x @ stacked()[0].t()) @ stacked()[1].t()
    y_ref.backward(g)
    want = [p.grad.clone() for pair in zip(As, Bs) for p in pair]
    want_x = x.grad.clone()
    for p in As + Bs + [x]:
        p.grad = None
    plan, r0 = [], 0
    for (s0, e0), r, sc in zip(rows, ranks, scal):
        plan.append((r0, r, s0, e0, sc))
        r0 += r
    params = [p for pair in zip(As, Bs) for p in pair]
    params[0].main_grad = torch.full_like(params[0], 7.0)          # one parameter with an optimizer bucket view
    with torch.no_grad():
        a_cat, b_bd = stacked()
    for rep in range(2):
        y = _LoRALinear.apply(x, w, a_cat, b_bd, None, tuple(plan), *params)
        y.backward(g)
    assert torch.allclose(y, y_ref, atol=1e-4)
    assert params[0].grad is None and torch.allclose(params[0].main_grad, 2 * want[0], atol=1e-4)   # overwrite + accumulate
    for p, wgt in list(zip(params, want))[1:]:
        assert torch.allclose(p.grad, 2 * wgt, atol=1e-4, rtol=1e-4)
    assert torch.allclose(x.grad, 2 * want_x, atol=1e-4)


def test_a_checkpoint_of_another_shape_is_refused_whole():
    """Shapes are checked for every tensor before the first copy: a checkpoint that does not fit raises, names the
    tensors, and leaves the model bit-identical; a missing key under ``strict`` does the same."""
    import copy as _copy
    import os
    import pytest
    from safetensors.torch import load_file, save_file
    with tempfile.TemporaryDirectory() as d:
        _full_model(d)
        wider = _copy.deepcopy(CFG)
        wider.intermediate_size = 128                       # only the MLP tensors differ; the embedding comes first and fits
        m = ParallelTransformerModel(wider)
        m.init_weights(11)
        before = [p.detach().clone() for p in m.parameters()]
        with pytest.raises(ValueError, match=r"mlp\.\{gate,up\}_proj\.weight.*nothing was loaded|nothing was loaded.*mlp"):
            load_from_hf_checkpoint(m, d)
        assert all(torch.equal(a, b) for a, b in zip(before, m.parameters()))
        # strict and a key missing from the file
        f = os.path.join(d, "model.safetensors")
        sd = load_file(f)
        del sd["model.layers.1.self_attn.o_proj.weight"]
        save_file(sd, f)
        fit = ParallelTransformerModel(CFG)
        fit.init_weights(12)
        before = [p.detach().clone() for p in fit.parameters()]
        with pytest.raises(KeyError):
            load_from_hf_checkpoint(fit, d, strict=True)
        assert all(torch.equal(a, b) for a, b in zip(before, fit.parameters()))
        loaded, missing = load_from_hf_checkpoint(fit, d)                  # tolerant: everything else is loaded
        assert missing == 1 and torch.equal(fit.layers[1].self_attn.o_proj.weight, before[[n for n, _ in fit.named_parameters()].index("layers.1.self_attn.o_proj.weight")])
        assert not torch.equal(fit.layers[0].self_attn.o_proj.weight, before[[n for n, _ in fit.named_parameters()].index("layers.0.self_attn.o_proj.weight")])
