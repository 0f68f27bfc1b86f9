"""3-D group layout, collectives, TP autograd regions and PP p2p over gloo on CPU."""
import torch

from _dist_util import run_ranks
from b200fw.dist.context import ParallelContext


def test_group_table_layout():
    tp, pp, dp = ParallelContext.group_table(8, tp=2, dp=2, pp=2)
    assert tp == [[0, 1], [2, 3], [4, 5], [6, 7]]
    assert pp == [[0, 2], [1, 3], [4, 6], [5, 7]]
    assert dp == [[0, 4], [1, 5], [2, 6], [3, 7]]
    assert ParallelContext.coords(5, tp=2, pp=2) == (1, 0, 1)
    tp, pp, dp = ParallelContext.group_table(8, tp=2, dp=4, pp=1)
    assert dp == [[0, 2, 4, 6], [1, 3, 5, 7]] and pp == [[r] for r in [0, 1, 2, 3, 4, 5, 6, 7]]


def _groups(rank, world):
    ctx = ParallelContext.init_distributed(tp_size=2, dp_size=2, pp_size=1, backend="gloo")
    return (ctx.tp_rank, ctx.dp_rank, ctx.tp_ranks, ctx.dp_ranks)


def test_process_groups_gloo():
    res = run_ranks(_groups, 4)
    assert res[0] == (0, 0, [0, 1], [0, 2]) and res[3] == (1, 1, [2, 3], [1, 3])


def _collectives(rank, world):
    from b200fw.dist import comm
    ctx = ParallelContext.init_distributed(tp_size=world, backend="gloo")
    g = ctx.tp_group
    x = torch.full((4, 3), float(rank + 1))
    assert torch.equal(comm.all_reduce(x.clone(), g), torch.full((4, 3), 3.0))
    ag = comm.all_gather(x, g)
    assert ag.shape == (8, 3) and ag[0, 0] == 1 and ag[4, 0] == 2
    assert comm.all_gather_last_dim(x, g).shape == (4, 6)
    rs = comm.reduce_scatter(torch.arange(8.0).reshape(4, 2) + rank, g)
    assert torch.equal(rs, (torch.arange(8.0).reshape(4, 2) * 2 + 1)[rank * 2:(rank + 1) * 2])
    b = torch.full((2,), float(rank))
    assert comm.broadcast(b, 1, g)[0] == 1
    # autograd regions
    a = torch.ones(2, 2, requires_grad=True)
    comm.copy_to_parallel_region(a, g).sum().backward()
    assert torch.equal(a.grad, torch.full((2, 2), 2.0))
    a = torch.ones(2, 2, requires_grad=True)
    y = comm.reduce_from_parallel_region(a * (rank + 1), g)
    assert torch.equal(y, torch.full((2, 2), 3.0))
    y.sum().backward()
    assert torch.equal(a.grad, torch.full((2, 2), float(rank + 1)))
    a = torch.ones(2, 2, requires_grad=True)
    y = comm.gather_from_parallel_region(a, g)
    (y * torch.arange(4.0)).sum().backward()
    assert torch.equal(a.grad[0], torch.tensor([0.0, 1.0]) + 2 * rank)
    # sequence-parallel pair
    a = torch.ones(2, 3, requires_grad=True)
    y = comm.gather_sequence(a * (rank + 1), g)
    assert y.shape == (4, 3)
    y.sum().backward()
    assert torch.equal(a.grad, torch.full((2, 3), 2.0 * (rank + 1)))
    # async all-reduce with bounded wait
    h = comm.AsyncAllReduce().launch(x.clone(), g)
    h.wait(timeout_sec=30)
    assert h.is_completed()
    return True


def test_collectives_and_regions():
    assert all(run_ranks(_collectives, 2))


def _p2p(rank, world):
    from b200fw.dist import comm
    ctx = ParallelContext.init_distributed(pp_size=world, backend="gloo")
    dev = torch.device("cpu")
    if rank == 0:
        comm.send_forward(torch.arange(6.0).reshape(2, 3), ctx.pp_next_rank, ctx.pp_group)
        g = comm.recv_backward((2, 3), torch.float32, dev, ctx.pp_next_rank, ctx.pp_group)
        assert torch.equal(g, torch.full((2, 3), 7.0))
        g2 = comm.send_forward_recv_backward(torch.ones(2, 3), (2, 3), torch.float32, dev, ctx.pp_next_rank, ctx.pp_group)
        assert torch.equal(g2, torch.full((2, 3), 9.0))
    else:
        x = comm.recv_forward((2, 3), torch.float32, dev, ctx.pp_prev_rank, ctx.pp_group)
        assert torch.equal(x, torch.arange(6.0).reshape(2, 3))
        comm.send_backward(torch.full((2, 3), 7.0), ctx.pp_prev_rank, ctx.pp_group)
        x2 = comm.send_backward_recv_forward(torch.full((2, 3), 9.0), (2, 3), torch.float32, dev, ctx.pp_prev_rank, ctx.pp_group)
        assert torch.equal(x2, torch.ones(2, 3))
    assert ctx.is_first_pp_stage == (rank == 0) and ctx.is_last_pp_stage == (rank == 1)
    return True


def test_pp_p2p():
    assert all(run_ranks(_p2p, 2))


def test_async_handle_timeout():
    from b200fw.dist.comm import AsyncHandle

    class Never:
        def is_completed(self):
            return False

        def wait(self):
            raise AssertionError("must not block")

    import pytest
    with pytest.raises(RuntimeError):
        AsyncHandle(work=Never()).wait(timeout_sec=0.05, poll_s=0.01)


def test_stream_manager_cpu_noop():
    from b200fw.dist.streams import StreamManager
    sm = StreamManager()
    with sm.comm_context():
        pass
    sm.sync_compute_to_comm()
    assert sm.get_stats()["comm_ops"] == 1


def test_destroy_runs_registered_callbacks_first():
    """Teardown hooks (release of CUDA graphs that captured collectives) run before the groups go, newest
    first, and a failing one does not stop the teardown."""
    ctx = ParallelContext.init_single_process()
    order = []
    ctx.on_destroy(lambda: order.append("a"))
    ctx.on_destroy(lambda: 1 / 0)
    ctx.on_destroy(lambda: order.append("b"))
    ctx.destroy()
    assert order == ["b", "a"] and ParallelContext._instance is None
    ctx.destroy()                                   # callbacks ran once
    assert order == ["b", "a"]


def _biased_tp_layers(rank, world):
    """Column- and row-parallel layers with a bias, a row layer fed the unsplit input, and the MLP built from plain
    sizes: each against ``nn.Linear`` holding the concatenated weights (outputs and input gradients)."""
    import torch.distributed as dist
    import torch.nn.functional as F
    from b200fw.dist import comm
    from b200fw.model.qwen3 import ColumnParallelLinear, ParallelMLP, RowParallelLinear
    ctx = ParallelContext.init_distributed(tp_size=world, backend="gloo")
    g = ctx.tp_group
    torch.manual_seed(7)                     # same stream on every rank: full reference weights
    w_col, b_col = torch.randn(24, 16) * 0.1, torch.randn(24)
    w_row, b_row = torch.randn(12, 24) * 0.1, torch.randn(12)
    x = torch.randn(3, 5, 16, requires_grad=True)
    xr = x.detach().clone().requires_grad_(True)

    col = ColumnParallelLinear(16, 24, ctx, bias=True, gather_output=True)
    row = RowParallelLinear(24, 12, ctx, bias=True, input_is_parallel=False)
    n_c, n_r = 24 // world, 24 // world
    with torch.no_grad():
        col.weight.copy_(w_col[rank * n_c:(rank + 1) * n_c]); col.bias.copy_(b_col[rank * n_c:(rank + 1) * n_c])
        row.weight.copy_(w_row[:, rank * n_r:(rank + 1) * n_r]); row.bias.copy_(b_row)
    y = row(col(x))                           # gathered column output -> row layer slices it again
    ref = F.linear(F.linear(xr, w_col, b_col), w_row, b_row)
    y.sum().backward(); ref.sum().backward()
    err = [(y - ref).abs().max().item(), (x.grad - xr.grad).abs().max().item(),
           (row.bias.grad - torch.full((12,), 15.0)).abs().max().item()]

    mlp = ParallelMLP(16, 32, ctx)
    assert mlp.gate_proj.weight.shape == (32 // world, 16) and mlp.up_proj.weight.shape == (32 // world, 16)
    parts = lambda t: [torch.empty_like(t) for _ in range(world)]
    gw, uw, dw = parts(mlp.gate_proj.weight.data), parts(mlp.up_proj.weight.data), parts(mlp.down_proj.weight.data)
    dist.all_gather(gw, mlp.gate_proj.weight.data.contiguous(), group=g)
    dist.all_gather(uw, mlp.up_proj.weight.data.contiguous(), group=g)
    dist.all_gather(dw, mlp.down_proj.weight.data.contiguous(), group=g)
    xm = torch.randn(2, 4, 16)
    out = mlp(xm)
    ref_m = F.linear(F.silu(F.linear(xm, torch.cat(gw, 0))) * F.linear(xm, torch.cat(uw, 0)), torch.cat(dw, 1))
    assert out.shape == ref_m.shape
    err.append((out - ref_m).abs().max().item())
    return err


def test_tp_layers_with_bias_and_unsplit_input():
    for err in run_ranks(_biased_tp_layers, 2):
        assert max(err) < 1e-5, err


def test_heartbeat_watcher_finds_a_silent_peer_and_an_announced_leave():
    """Three watchers on one in-process store, driven by hand with a made-up clock: beats keep everybody alive; a
    peer whose counter stands still longer than the limit is reported with its rank; an announced leave is reported at
    the next look, with the reason; ``check()`` is quiet until then and raises the same error ever after."""
    import pytest
    import torch.distributed as dist
    from b200fw.dist import PeerLostError, RankHeartbeat
    store = dist.HashStore()
    hb = [RankHeartbeat(store, r, 3, interval_s=1.0, timeout_s=5.0) for r in range(3)]
    t = 100.0
    for step in range(8):                       # everyone beats: nobody is lost
        for h in hb:
            h.beat()
        for h in hb:
            h.poll(now=t)
            h.check()
        t += 1.0
    for step in range(7):                       # rank 2 goes silent
        hb[0].beat()
        hb[1].beat()
        hb[0].poll(now=t)
        hb[1].poll(now=t)
        t += 1.0
    for h in hb[:2]:
        with pytest.raises(PeerLostError) as e:
            h.check()
        assert e.value.rank == 2 and "no heartbeat" in e.value.reason
        with pytest.raises(PeerLostError):
            h.check()                           # and it stays raised
    # an announced leave is seen at once, whatever the clock says
    store2 = dist.HashStore()
    a, b = RankHeartbeat(store2, 0, 2, 1.0, 5.0), RankHeartbeat(store2, 1, 2, 1.0, 5.0)
    a.beat(); b.beat(); a.poll(now=0.0); a.check()
    b.announce_leave("out of memory on this rank")
    a.poll(now=0.1)
    with pytest.raises(PeerLostError, match="announced its leave: out of memory"):
        a.check()
    # a peer that never wrote a beat counts from the first look (a rank that died before its first beat)
    store3 = dist.HashStore()
    c = RankHeartbeat(store3, 0, 2, 1.0, 5.0)
    c.poll(now=0.0)
    c.poll(now=4.0)
    c.check()
    c.poll(now=6.0)
    with pytest.raises(PeerLostError):
        c.check()


def test_heartbeat_thread_beats_polls_and_stops():
    import time
    import torch.distributed as dist
    from b200fw.dist import RankHeartbeat
    store = dist.HashStore()
    a = RankHeartbeat(store, 0, 2, interval_s=0.02, timeout_s=1.0).start()       # generous limit: a loaded test box
    b = RankHeartbeat(store, 1, 2, interval_s=0.02, timeout_s=1.0).start()       # may starve a thread for a while
    time.sleep(0.3)
    a.check(); b.check()
    assert a.beats > 5 and b.beats > 5
    b.stop()                                    # b goes silent without a word
    deadline = time.time() + 10
    while a.lost is None and time.time() < deadline:
        time.sleep(0.02)
    assert a.lost is not None and a.lost.rank == 1
    a.stop()
    assert a._thread is None
