"""Property test (hypothesis) of the bucketed ZeRO optimizer on one process: for random parameter shapes, bucket sizes,
stages, accumulation lengths, clipping thresholds and hyper-parameters the result equals ``torch.optim.AdamW`` with
``clip_grad_norm_``; a non-finite gradient skips the update and leaves every state untouched."""
import pytest
import torch

hypothesis = pytest.importorskip("hypothesis")
from hypothesis import given, settings  # noqa: E402
from hypothesis import strategies as st  # noqa: E402

from b200fw.optim import build_optimizer  # noqa: E402

SHAPES = st.lists(st.one_of(st.tuples(st.integers(1, 9)), st.tuples(st.integers(1, 7), st.integers(1, 7))), min_size=1, max_size=6)


@settings(max_examples=120, deadline=None)
@given(SHAPES, st.sampled_from([0, 1, 2, 3]), st.integers(1, 3), st.sampled_from([1e-5, 2e-4, 1.0]),
       st.sampled_from([0.0, 0.3, 1e9]), st.sampled_from([1e-3, 5e-2]), st.sampled_from([0.0, 0.1]), st.integers(0, 10 ** 6))
def test_bucketed_optimizer_equals_adamw(shapes, stage, accum, bucket_mb, max_norm, lr, wd, seed):
    g = torch.Generator().manual_seed(seed)
    params = [torch.nn.Parameter(torch.randn(*sh, generator=g)) for sh in shapes]
    ref = [torch.nn.Parameter(p.detach().clone()) for p in params]
    opt = build_optimizer(params, stage, lr=lr, weight_decay=wd, bucket_mb=bucket_mb)
    ropt = torch.optim.AdamW(ref, lr=lr, weight_decay=wd)
    for step in range(3):
        for a in range(accum):
            opt.pre_forward()
            opt.begin_backward(sync=a == accum - 1)
            grads = [torch.randn(*sh, generator=g) for sh in shapes]
            # a loss whose gradient w.r.t. every parameter is the drawn tensor (parameters are bound to buckets here)
            sum((p * gr).sum() for p, gr in zip(params, grads)).backward()
            for r, gr in zip(ref, grads):
                r.grad = gr.clone() if r.grad is None else r.grad + gr
            opt.post_backward()
        gn = float(opt.clip_grad_norm(max_norm if max_norm > 0 else None))
        want = float(torch.nn.utils.clip_grad_norm_(ref, max_norm if max_norm > 0 else float("inf")))
        assert abs(gn - want) <= 1e-4 * max(1.0, want)
        opt.step()
        opt.zero_grad()
        ropt.step()
        ropt.zero_grad()
        with opt.eval_mode():
            for p, r in zip(params, ref):
                assert torch.allclose(p.detach(), r.detach(), atol=2e-5, rtol=2e-5), (step, stage)
    # a non-finite gradient: the step is skipped, parameters and moments stay as they are
    with opt.eval_mode():
        before = [p.detach().clone() for p in params]
    m_before, v_before = opt.exp_avg.clone(), opt.exp_avg_sq.clone()
    opt.pre_forward()
    opt.begin_backward(sync=True)
    sum((p * float("nan")).sum() for p in params).backward()
    opt.post_backward()
    assert float(opt.clip_grad_norm(1.0)) < 0
    opt.step()
    opt.zero_grad()
    with opt.eval_mode():
        assert all(torch.equal(a, p.detach()) for a, p in zip(before, params))
    assert torch.equal(m_before, opt.exp_avg) and torch.equal(v_before, opt.exp_avg_sq)
