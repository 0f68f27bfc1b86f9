"""Multi-GPU paths (need >= 2 GPUs): flag barrier, ZeRO with in-kernel peer reduce-scatter / all-gather
against the NCCL path, peer-write weight sync across GPUs, fused tensor-parallel GEMM kernels."""
import pytest
import torch

pytestmark = pytest.mark.gpu

needs2 = pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2,
                            reason="needs at least 2 GPUs")


def _world():
    return min(torch.cuda.device_count(), 8)


def _flag_worker(rank, world):
    import torch.distributed as dist
    from b200fw.dist.symm import FlagBarrier, SymmetricBuffer
    g = dist.group.WORLD
    fb = FlagBarrier(g, limit_ms=2000)
    buf = SymmetricBuffer(1024, torch.float32, g)
    ok = True
    for it in range(1, 6):
        buf.tensor.fill_(float(rank * 100 + it))
        fb.barrier(0)
        # read every peer's buffer through its pointer (a device-to-device copy from peer memory)
        for r in range(world):
            peer = torch.empty(1024, device="cuda")
            torch.cuda.current_stream().synchronize()
            import ctypes
            from b200fw import _native as nv
            nv.check(nv.lib().b2_peer_write(ctypes.c_void_p(buf.peer_ptrs[r]), 1, nv.ptr(peer), 1,
                                            ctypes.c_longlong(1024), ctypes.c_longlong(0), 0, nv.ptr(None),
                                            nv.stream_ptr()), "peer_read")
            ok = ok and bool((peer == float(r * 100 + it)).all())
        fb.barrier(1)
    return ok and fb.ok()


@needs2
def test_flag_barrier_and_peer_pointers():
    from _gpu_dist_util import run_gpu_ranks
    assert all(run_gpu_ranks(_flag_worker, _world()))


def _wait_timeout_worker(rank, world):
    """A wait on a flag nobody sets runs out after its limit and reports through the status word; the
    context stays usable afterwards."""
    import torch.distributed as dist
    from b200fw import _native as nv
    from b200fw.dist.symm import FlagBarrier
    fb = FlagBarrier(dist.group.WORLD, limit_ms=300)
    fb.wait(channel=3, epoch=7)                 # no rank ever signals channel 3
    ok_before = fb.ok()
    status = nv.read_status()                   # reads and clears
    x = torch.ones(8, device="cuda") * 2        # the device still works
    fb.barrier(0)
    return (ok_before, status, float(x.sum()), fb.ok())


@needs2
def test_bounded_wait_reports_instead_of_hanging():
    from _gpu_dist_util import run_gpu_ranks
    for ok_before, status, s, ok_after in run_gpu_ranks(_wait_timeout_worker, 2):
        assert ok_before is False and status == 301 and s == 16.0 and ok_after is True


def _zero_worker(rank, world, backend, stage):
    from b200fw.train import TrainConfig, TrainEngine
    cfg = TrainConfig(model_preset="tiny128", dp_size=world, lora_rank=0, grpo_beta=0.0, learning_rate=1e-3,
                      gradient_accumulation_steps=2, zero_stage=stage, warmup_steps=0, max_seq_len=256,
                      amp_dtype="bf16", zero_comm_backend=backend, bucket_mb=1.0)
    eng = TrainEngine(cfg).initialize()
    assert eng.optimizer.p2p == (backend == "p2p")
    import os
    if backend == "p2p" and os.environ.get("B200FW_NVLS") == "0":
        assert not eng.optimizer.nvls
    if backend == "p2p" and os.environ.get("B200FW_ZERO_NVLS") == "1" and eng.optimizer.buckets[0].symm_grad.mc_ptr:
        assert eng.optimizer.nvls
    out = []
    for s in range(6):
        g = torch.Generator().manual_seed(s * 31 + rank)
        ids = torch.randint(0, 8192, (2, 256), generator=g)
        labels = ids.clone()
        labels[:, :128] = -100
        m = eng.sft_step_tensors(ids, labels)
        out.append((m.loss, m.grad_norm))
    flat = torch.cat([p.detach().float().reshape(-1) for p in eng.model.parameters()])
    return out, float(flat.double().sum()), float(flat.abs().double().sum())


@needs2
@pytest.mark.parametrize("stage,nvls", [(1, "1"), (2, "1"), (1, "0")])
def test_zero_p2p_matches_nccl(stage, nvls):
    """The in-kernel data plane (per-bucket device barrier + reduce launched from the gradient hooks, one-kernel
    norm exchange, AdamW + publish, end-of-step barrier) against NCCL reduce-scatter / all-gather; with the
    switch's multimem reduce / store where the platform offers it (nvls "1") and with plain peer loads / stores."""
    from _gpu_dist_util import run_gpu_ranks
    w = _world()
    a = run_gpu_ranks(_zero_worker, w, "nccl", stage)
    # B200FW_ZERO_NVLS forces the multimem reduce / publish kernels on (or off) whatever the rank count: the automatic
    # choice keeps them for more than two ranks
    b = run_gpu_ranks(_zero_worker, w, "p2p", stage, env={"B200FW_NVLS": nvls, "B200FW_ZERO_NVLS": nvls})
    for r in range(w):
        assert a[r][1] == a[0][1] and b[r][1] == b[0][1]            # ranks hold identical weights
        for i, ((la, ga), (lb, gb)) in enumerate(zip(a[r][0], b[r][0])):
            assert abs(la - lb) < 5e-2, (i, la, lb)
            if i < 2:     # later steps amplify bf16 rounding differences between the two reduction orders
                assert abs(ga - gb) / max(ga, 1e-6) < 5e-2, (i, ga, gb)
        assert abs(a[r][2] - b[r][2]) / a[r][2] < 2e-3


def _zero_symm_failure_worker(rank, world):
    from b200fw.optim import zero
    from b200fw.train import TrainConfig, TrainEngine
    real = zero.ZeROOptimizer._make_symmetric

    def broken(self):
        real(self)                      # the collective part (rendezvous) runs on every rank
        if rank == world - 1:
            raise RuntimeError("set-up failed on this rank after the rendezvous (made up by the test)")
    zero.ZeROOptimizer._make_symmetric = broken
    cfg = TrainConfig(model_preset="tiny128", dp_size=world, lora_rank=0, grpo_beta=0.0, learning_rate=1e-3,
                      gradient_accumulation_steps=1, zero_stage=1, warmup_steps=0, max_seq_len=128,
                      amp_dtype="bf16", zero_comm_backend="auto", bucket_mb=1.0)
    import warnings
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        eng = TrainEngine(cfg).initialize()
    assert not eng.optimizer.p2p and eng.optimizer.comm_backend == "nccl" and eng.optimizer.flags is None
    losses = []
    ids = torch.randint(0, 8192, (2, 128), generator=torch.Generator().manual_seed(7 + rank))
    for s in range(4):                  # the same batch every step: the loss on it must fall
        losses.append(eng.sft_step_tensors(ids, ids.clone()).loss)
    flat = torch.cat([p.detach().float().reshape(-1) for p in eng.model.parameters()])
    return losses, float(flat.double().sum())


@needs2
def test_zero_auto_backend_falls_back_together_when_one_rank_has_no_symmetric_memory():
    """The failure is made on the host (an exception in one rank's set-up); every rank must end up on the NCCL path,
    hold identical weights and make progress."""
    from _gpu_dist_util import run_gpu_ranks
    w = _world()
    out = run_gpu_ranks(_zero_symm_failure_worker, w)
    assert all(out[r][1] == out[0][1] for r in range(w))
    assert out[0][0][-1] < out[0][0][0]


def _zero_wait_runs_out_worker(rank, world):
    """Rank 0 waits (300 ms limit) on a barrier channel that rank 1 never enters: the wait runs out, the device-side
    ``ok`` word is cleared, this step's AdamW leaves rank 0's shard untouched, and the host raises at the step's
    sync instead of training on.  Nothing faults; both ranks finish the step's collectives and leave between steps."""
    from b200fw import _native as nv
    from b200fw.train import TrainConfig, TrainEngine
    cfg = TrainConfig(model_preset="tiny128", dp_size=world, lora_rank=0, grpo_beta=0.0, learning_rate=1e-3,
                      gradient_accumulation_steps=1, zero_stage=1, warmup_steps=0, max_seq_len=256,
                      amp_dtype="bf16", zero_comm_backend="p2p", bucket_mb=1.0)
    eng = TrainEngine(cfg).initialize()
    opt = eng.optimizer
    g = torch.Generator().manual_seed(rank)
    ids = torch.randint(0, 8192, (2, 256), generator=g)
    labels = ids.clone()
    labels[:, :128] = -100
    eng.sft_step_tensors(ids, labels)                    # a clean step first
    before = opt.master.clone()
    raised = False
    if rank == 0:
        keep = opt.flags.limit_ms
        opt.flags.limit_ms = 300
        opt.flags.barrier_dev(opt._ch_spare)             # nobody else signals this channel
        opt.flags.limit_ms = keep
    try:
        eng.sft_step_tensors(ids, labels)
    except nv.NativeError as e:
        raised = "301" in str(e)
    torch.cuda.synchronize()
    unchanged = bool(torch.equal(opt.master, before))
    alive = float((torch.ones(4, device="cuda") * 3).sum())
    return raised, unchanged, alive


@needs2
def test_zero_p2p_wait_that_runs_out_skips_the_update_and_raises():
    from _gpu_dist_util import run_gpu_ranks
    r0, r1 = run_gpu_ranks(_zero_wait_runs_out_worker, 2, env={"B200FW_NVLS": "0"})
    assert r0 == (True, True, 12.0)                      # raised, shard untouched, device usable
    assert r1 == (False, False, 12.0)                    # the healthy rank stepped normally


def _zero3_worker(rank, world, stage):
    from b200fw.train import TrainConfig, TrainEngine
    cfg = TrainConfig(model_preset="tiny128", dp_size=world, lora_rank=0, grpo_beta=0.0, learning_rate=1e-3,
                      gradient_accumulation_steps=2, zero_stage=stage, warmup_steps=0, max_seq_len=256,
                      amp_dtype="bf16", bucket_mb=1.0)
    eng = TrainEngine(cfg).initialize()
    hooks = len(eng.optimizer._prefetch_hooks)
    out = []
    for s in range(5):
        g = torch.Generator().manual_seed(s * 31 + rank)
        ids = torch.randint(0, 8192, (2, 256), generator=g)
        labels = ids.clone()
        labels[:, :128] = -100
        m = eng.sft_step_tensors(ids, labels)
        out.append((m.loss, m.grad_norm))
    with eng.optimizer.eval_mode():
        flat = torch.cat([p.detach().float().reshape(-1) for p in eng.model.parameters()])
        res = float(flat.double().sum()), float(flat.abs().double().sum())
    return out, res, hooks, len(eng.optimizer.buckets)


@needs2
def test_zero3_prefetched_gathers_match_zero1():
    """ZeRO-3 with the parameter gathers queued on the side stream and waited for layer by layer trains
    like ZeRO-1 (same data, same seeds)."""
    from _gpu_dist_util import run_gpu_ranks
    w = min(_world(), 2)
    a = run_gpu_ranks(_zero3_worker, w, 1)
    b = run_gpu_ranks(_zero3_worker, w, 3)
    assert b[0][2] > 1 and b[0][3] > 2 and a[0][2] == 0            # hooks installed at stage 3 only; several buckets
    for r in range(w):
        assert b[r][1] == b[0][1]                                    # ranks hold identical weights
        for i, ((la, ga), (lb, gb)) in enumerate(zip(a[r][0], b[r][0])):
            assert abs(la - lb) < 5e-2, (i, la, lb)
            if i < 2:
                assert abs(ga - gb) / max(ga, 1e-6) < 5e-2, (i, ga, gb)
        assert abs(a[r][1][1] - b[r][1][1]) / a[r][1][1] < 2e-3


def _graph_dp_worker(rank, world, graph, reduce_in_graph, backend="nccl"):
    from b200fw.train import TrainConfig, TrainEngine
    cfg = TrainConfig(model_preset="tiny128", dp_size=world, lora_rank=0, grpo_beta=0.0, learning_rate=1e-3,
                      gradient_accumulation_steps=2, zero_stage=1, warmup_steps=0, max_seq_len=256, amp_dtype="bf16",
                      bucket_mb=1.0, cuda_graph_step=graph, cuda_graph_reduce=reduce_in_graph,
                      zero_comm_backend=backend)
    eng = TrainEngine(cfg).initialize()
    assert eng.optimizer.comm_backend == ("p2p" if backend in ("p2p", "auto") else "nccl")
    out = []
    for s in range(14):                      # 7 optimizer steps: two eager occurrences per graph key, then replays
        g = torch.Generator().manual_seed(s * 31 + rank)
        ids = torch.randint(0, 8192, (2, 256), generator=g)
        labels = ids.clone()
        labels[:, :128] = -100
        m = eng.sft_step_tensors(ids, labels)
        out.append((m.loss, m.grad_norm))
    flat = torch.cat([p.detach().float().reshape(-1) for p in eng.model.parameters()])
    keys = sorted(k[3:] for k in eng._graphs)
    return out, float(flat.double().sum()), float(flat.abs().double().sum()), keys, eng._graph_disabled


@needs2
@pytest.mark.parametrize("backend", ["nccl", "auto"])
def test_graphed_micro_step_with_captured_reduce_scatter_matches_eager(backend):
    """Data parallel: the last micro-batch's graph contains the bucket reduce-scatters (side stream forked
    and joined inside the capture); losses, gradient norms and weights follow the eager NCCL run.  With the
    default ("auto") backend the captured reductions are the in-kernel ones: device-epoch barrier + peer /
    multimem reduce per bucket."""
    from _gpu_dist_util import run_gpu_ranks
    w = min(_world(), 2) if backend == "nccl" else _world()
    eager = run_gpu_ranks(_graph_dp_worker, w, False, False, "nccl")
    fused = run_gpu_ranks(_graph_dp_worker, w, True, True, backend)
    plain = run_gpu_ranks(_graph_dp_worker, w, True, False, backend)
    assert fused[0][3] == [(False, True), (True, False)] and not fused[0][4]       # (first, reduce captured) keys
    assert plain[0][3] == [(False, False), (True, False)] and eager[0][3] == []
    for r in range(w):
        for other in (fused, plain):
            assert other[r][1] == other[0][1]                                     # ranks hold identical weights
            for i, ((la, ga), (lb, gb)) in enumerate(zip(eager[r][0], other[r][0])):
                assert abs(la - lb) < 2e-2, (i, la, lb)
                assert (ga > 0) == (i % 2 == 1) and (gb > 0) == (ga > 0)          # every second micro-batch steps
                if ga > 0 and i < 8:   # later steps amplify the rounding noise of atomically accumulated gradients
                    assert abs(ga - gb) / ga < 5e-2, (i, ga, gb)
            assert abs(eager[r][2] - other[r][2]) / eager[r][2] < 1e-3


def _peer_sync_worker(rank, world):
    import torch.distributed as dist
    from b200fw.sync import PeerWeightSync
    layout = [("w1", (513, 257)), ("w2", (1000,)), ("w3", (64, 64))]
    ps = PeerWeightSync(layout, torch.bfloat16, group=dist.group.WORLD, sender_rank=0)
    got = {}

    class Eng:
        def load_weights(self, views):
            got.update({k: v.clone() for k, v in views.items()})

    g = torch.Generator().manual_seed(5)
    state = {k: torch.empty(shape).normal_(generator=g).cuda() for k, shape in layout}   # fp32 source: cast in flight
    v1 = ps.sync(rank == 0, state if rank == 0 else None, None if rank == 0 else Eng())
    ok1 = rank == 0 or all(torch.equal(got[k], state[k].to(torch.bfloat16)) for k in state)
    got.clear()
    v2 = ps.sync(rank == 0, {k: v * 2 for k, v in state.items()} if rank == 0 else None,
                 None if rank == 0 else Eng(), corrupt=True)
    rej = ps.get_stats()["rejected"]
    # delta on one tensor: verified over the spans it touched; a corrupted delta is rejected as well
    v3 = ps.sync(rank == 0, state if rank == 0 else None, None if rank == 0 else Eng())       # clean image
    got.clear()
    delta = {"w2": torch.ones(1000, device="cuda")}
    v4 = ps.sync(rank == 0, delta if rank == 0 else None, None if rank == 0 else Eng(), add=True)
    ok4 = rank == 0 or torch.equal(got["w2"], (state["w2"].to(torch.bfloat16).float() + 1).to(torch.bfloat16))
    got.clear()
    v5 = ps.sync(rank == 0, delta if rank == 0 else None, None if rank == 0 else Eng(), add=True, corrupt=True)
    return v1, ok1, v2, len(got), rej, (v3, v4, ok4, v5, ps.get_stats()["rejected"])


@needs2
def test_peer_write_weight_sync_across_gpus():
    from _gpu_dist_util import run_gpu_ranks
    res = run_gpu_ranks(_peer_sync_worker, 2)
    assert res[0][:3] == (1, True, 1) and res[1][:4] == (1, True, 1, 0) and res[1][4] == 1
    assert res[0][5][:4] == (2, 3, True, 3) and res[1][5] == (2, 3, True, 3, 2)


def _fused_tp_ops_worker(rank, world):
    import torch.distributed as dist
    from b200fw.ops import fused_tp
    g = dist.group.WORLD
    torch.manual_seed(7)                       # same "global" tensors on every rank
    results = []
    for (rows, K, N, b_mn) in [(256, 512, 768, False), (128, 1024, 256, True), (256, 512, 768, False), (384, 264, 1024, False)]:
        M = rows * world
        for rep in range(3):                   # repeated calls exercise buffer parity and epochs
            x_full = torch.randn(M, K * world, device="cuda", dtype=torch.bfloat16) * 0.5
            w_full = torch.randn(N, K * world, device="cuda", dtype=torch.bfloat16) * 0.1
            res_full = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
            # ---- GEMM -> reduce-scatter: K is sharded, rows are scattered
            xl = x_full[:, rank * K:(rank + 1) * K].contiguous()
            wl = w_full[:, rank * K:(rank + 1) * K].contiguous()
            w_arg = wl.t().contiguous() if b_mn else wl
            res_l = res_full[rank * rows:(rank + 1) * rows].contiguous()
            got = fused_tp.gemm_reduce_scatter(xl, w_arg, g, b_mn=b_mn, residual=res_l)
            want = (x_full.float() @ w_full.float().t() + res_full.float())[rank * rows:(rank + 1) * rows]
            e1 = ((got.float() - want).abs().max() / want.abs().max()).item()
            # ---- all-gather -> GEMM: rows are sharded, N is local
            xs = x_full[rank * rows:(rank + 1) * rows, :K].contiguous()
            wn = w_full[:, :K].contiguous()
            # odd repetitions use a call-site slot: the gathered activations are then the buffer itself (no copy)
            y, xg = fused_tp.allgather_gemm(xs, wn.t().contiguous() if b_mn else wn, g, b_mn=b_mn,
                                            slot="test" if rep % 2 else None)
            want_y = x_full[:, :K].float() @ wn.float().t()
            e2 = ((y.float() - want_y).abs().max() / want_y.abs().max()).item()
            e3 = float((xg != x_full[:, :K]).sum())
            results.append((e1, e2, e3))
    return results


@needs2
@pytest.mark.parametrize("nvls", ["1", "0"])
def test_fused_tp_gemm_kernels_match_reference(nvls):
    """GEMM -> reduce-scatter and all-gather -> GEMM against fp32 matmuls of the full tensors, on every visible GPU
    (2, 4 or 8); the all-gather pushes through the switch's multicast address (nvls "1", where the platform has it)
    or with one store per peer (nvls "0")."""
    from _gpu_dist_util import run_gpu_ranks
    for res in run_gpu_ranks(_fused_tp_ops_worker, _world() if _world() in (2, 4, 8) else 2, env={"B200FW_NVLS": nvls}):
        for e1, e2, e3 in res:
            assert e1 < 2e-2 and e2 < 2e-2 and e3 == 0.0, (e1, e2, e3)


def _vocab_parallel_worker(rank, world):
    import torch.distributed as dist
    from b200fw.ops import VocabShard, lm_head_cross_entropy, lm_head_logprob
    torch.manual_seed(11)
    M, H, V = 384, 256, 4096
    h0 = (torch.randn(M, H, device="cuda") * 0.5).bfloat16()
    w0 = (torch.randn(V, H, device="cuda") * 0.05).bfloat16()
    labels = torch.randint(0, V, (M,), device="cuda")
    labels[::5] = -100
    vl = V // world
    out = []
    for fn in ("ce", "logp"):
        h = h0.clone().requires_grad_(True)
        w = w0.clone().requires_grad_(True)
        hs = h0.clone().requires_grad_(True)
        ws = w0[rank * vl:(rank + 1) * vl].clone().requires_grad_(True)
        shard = VocabShard(dist.group.WORLD, rank, world, V)
        if fn == "ce":
            a = lm_head_cross_entropy(h, w, labels, chunk=128)
            b = lm_head_cross_entropy(hs, ws, labels, chunk=128, shard=shard)
            a.backward()
            b.backward()
            e0 = (a - b).abs().item()
        else:
            a = lm_head_logprob(h, w, labels, temperature=0.9, chunk=128)
            b = lm_head_logprob(hs, ws, labels, temperature=0.9, chunk=128, shard=shard)
            gsel = torch.randn(M, device="cuda")
            (a * gsel).sum().backward()
            (b * gsel).sum().backward()
            e0 = (a - b).abs().max().item()
        e1 = ((h.grad.float() - hs.grad.float()).abs().max() / h.grad.float().abs().max()).item()
        e2 = ((w.grad.float()[rank * vl:(rank + 1) * vl] - ws.grad.float()).abs().max()
              / w.grad.float().abs().max()).item()
        out.append((e0, e1, e2))
    return out


@needs2
def test_vocab_parallel_lm_head_matches_replicated():
    from _gpu_dist_util import run_gpu_ranks
    for res in run_gpu_ranks(_vocab_parallel_worker, 2):
        for e0, e1, e2 in res:
            assert e0 < 5e-3 and e1 < 3e-2 and e2 < 3e-2, res


def _tp_train_worker(rank, world, fused):
    from b200fw.model import ModelConfig
    from b200fw.train import TrainConfig, TrainEngine
    mc = ModelConfig(vocab_size=8192, hidden_size=256, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=128,
                     intermediate_size=768, max_position_embeddings=4096, tie_word_embeddings=False)
    cfg = TrainConfig(model_config=mc, tp_size=world, lora_rank=0, grpo_beta=0.0, learning_rate=1e-3,
                      gradient_accumulation_steps=1, zero_stage=1, warmup_steps=0, max_seq_len=256, amp_dtype="bf16",
                      sequence_parallel=True, fused_tp_comm=fused)
    eng = TrainEngine(cfg).initialize()
    out = []
    for s in range(5):
        g = torch.Generator().manual_seed(s)
        ids = torch.randint(0, 8192, (2, 256), generator=g)
        labels = ids.clone()
        labels[:, :128] = -100
        m = eng.sft_step_tensors(ids, labels)
        out.append((m.loss, m.grad_norm))
    return out


@needs2
def test_tp_sequence_parallel_training_fused_vs_nccl():
    from _gpu_dist_util import run_gpu_ranks
    a = run_gpu_ranks(_tp_train_worker, 2, False)
    b = run_gpu_ranks(_tp_train_worker, 2, True)
    for x in (a, b):                                       # TP ranks agree (fp32 atomics reorder the loss sum)
        assert all(abs(p[0] - q[0]) < 1e-3 and abs(p[1] - q[1]) < 1e-3 for p, q in zip(x[0], x[1]))
    for (la, ga), (lb, gb) in zip(a[0], b[0]):
        assert abs(la - lb) < 5e-2 and abs(ga - gb) / max(ga, 1e-6) < 8e-2, (a[0], b[0])
    assert b[0][-1][0] < b[0][0][0] + 0.5


def _pp_train_worker(rank, world, pp):
    from b200fw.model import ModelConfig
    from b200fw.train import TrainConfig, TrainEngine
    mc = ModelConfig(vocab_size=8192, hidden_size=256, num_layers=4, num_heads=4, num_kv_heads=2, head_dim=128,
                     intermediate_size=768, max_position_embeddings=4096, tie_word_embeddings=False)
    cfg = TrainConfig(model_config=mc, pp_size=pp, num_micro_batches=4, lora_rank=0, grpo_beta=0.0, learning_rate=1e-3,
                      gradient_accumulation_steps=1, zero_stage=1, warmup_steps=0, max_seq_len=256, amp_dtype="bf16")
    eng = TrainEngine(cfg).initialize()
    out = []
    for s in range(5):
        g = torch.Generator().manual_seed(s)
        ids = torch.randint(0, 8192, (8, 256), generator=g)
        labels = ids.clone()
        labels[:, :128] = -100
        if pp > 1:
            m = eng.sft_step_tensors(ids, labels)
        else:                                    # the same 8 sequences as 4 accumulated micro-batches of 2
            eng.config.gradient_accumulation_steps = 4
            for k in range(4):
                m = eng.sft_step_tensors(ids[2 * k:2 * k + 2], labels[2 * k:2 * k + 2])
        out.append((m.loss, m.grad_norm))
    return out


@needs2
def test_pipeline_1f1b_with_prefetched_transfers_matches_one_gpu():
    """1F1B over two stages, activations and gradients on their own communicators and streams, receives posted one
    compute phase ahead: the loss curve follows the single-GPU run of the same micro-batches."""
    from _gpu_dist_util import run_gpu_ranks
    one = run_gpu_ranks(_pp_train_worker, 1, 1)[0]
    two = run_gpu_ranks(_pp_train_worker, 2, 2)
    # (losses are not compared: the single-GPU run reports its last micro-batch, the pipeline the mean over four)
    assert all(abs(l - 9.0) < 0.5 for l, _ in two[0])                 # random-init loss ~ ln(8192)
    for (l1, g1), (l2, g2) in zip(two[0], two[1]):
        assert abs(l1 - l2) < 1e-3 and abs(g1 - g2) < 1e-3            # both stages report the same numbers
    for i, ((_, ga), (_, gb)) in enumerate(zip(one, two[0])):
        if i < 2:
            assert abs(ga - gb) / max(ga, 1e-6) < 8e-2, (i, ga, gb)   # same gradients -> same global norm
