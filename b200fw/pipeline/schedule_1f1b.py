"""1F1B pipeline schedule.

Semantics of the reference scheduler (src/distributed/pipeline_scheduler.py:68-320): ``pp-1-rank``
warm-up forwards, steady one-forward-one-backward with combined send/recv pairs (which cannot
deadlock), cool-down backwards; each micro-batch's loss is scaled by ``1/num_micro``; a one-time
``int64[3]`` shape handshake travels stage to stage; received activations become autograd leaves.
Gradients accumulate into the optimizer's bucket buffers across micro-batches.

Transfers: activations and gradients use one communicator and one CUDA stream per direction
(:class:`b200fw.dist.comm.PipeChannel`); sends are queued behind the compute that produced their data and never hold
the compute stream (a stage goes straight on to its next micro-batch), receives land in persistent ring buffers and
are posted where their data is used.
"""
from __future__ import annotations

from collections import deque
from typing import Optional, Tuple

import torch
import torch.distributed as dist

from ..dist import comm


def default_loss_fn(logits: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
    """Token-mean cross-entropy of ``[*, V]`` logits against ``[*]`` labels, no next-token shift
    (src/distributed/pipeline_scheduler.py:55-65).  The scheduler itself uses the model's fused LM-head loss, which
    never materialises the logits; this function is the plain form for callers that already have them."""
    return torch.nn.functional.cross_entropy(logits.reshape(-1, logits.shape[-1]).float(), labels.reshape(-1).long())


class PipelineScheduler:
    def __init__(self, model, pp_context=None, num_micro_batches: Optional[int] = None, loss_fn=None):
        """``PipelineScheduler(model, pp_context, num_micro_batches)``; or, in the reference's form
        (src/distributed/pipeline_scheduler.py:82-103), ``PipelineScheduler(pp_context, num_micro_batches,
        loss_fn=None)`` with the stage model handed to :meth:`run_1f1b_schedule`.  With a ``loss_fn(logits, labels)``
        the last stage materialises its logits and calls it; without one it uses the model's fused next-token loss."""
        from .stages import PipelineParallelContext
        if isinstance(model, PipelineParallelContext):
            model, pp_context, num_micro_batches = None, model, (pp_context if num_micro_batches is None
                                                                else num_micro_batches)
        assert pp_context is not None and num_micro_batches is not None
        assert num_micro_batches >= pp_context.pp_size, "need num_micro_batches >= pp_size to fill the pipe"
        self.model, self.pp, self.num_micro = model, pp_context, int(num_micro_batches)
        self.loss_fn = loss_fn
        self._act_shape: Optional[Tuple[int, ...]] = None
        self.timeline = None  # optional ScheduleVisualizer
        self._fifo: deque = deque()   # (input, output) pairs queued by forward_step for backward_step

    # ---- shape handshake ---------------------------------------------------------------------------
    def _handshake(self, mb_tokens: int, device, dtype):
        if self._act_shape is not None and self._act_shape[0] * (self.model.tp_size if self.model.sequence_parallel else 1) == mb_tokens:
            return
        H = self.model.cfg.hidden_size
        if self.pp.is_first_stage:
            rows = mb_tokens // self.model.tp_size if self.model.sequence_parallel else mb_tokens
            shape = torch.tensor([rows, H, 0], dtype=torch.int64, device=device)
        else:
            shape = comm.recv_forward((3,), torch.int64, device, self.pp.prev_rank, self.pp.group)
        if not self.pp.is_last_stage:
            comm.send_forward(shape, self.pp.next_rank, self.pp.group)
        self._act_shape = (int(shape[0]), int(shape[1]))

    # ---- one micro-batch ---------------------------------------------------------------------------
    def _forward(self, ids_mb, labels_mb, recv):
        B, S = labels_mb.shape
        if self.pp.is_first_stage:
            inp = None
            out = self.model.forward_hidden(ids_mb, B, S)
        else:
            inp = recv.detach().requires_grad_(True)     # a fresh leaf over the (reused) receive buffer
            out = self.model.forward_hidden(inp, B, S)
        if self.pp.is_last_stage:
            if self.loss_fn is not None:
                logits = self.model.logits_from_hidden(out).reshape(B, S, -1)
                loss = self.loss_fn(logits, labels_mb) / self.num_micro
                return inp, loss, loss.detach()
            loss = self.model.loss(None, labels_mb, loss_scale=1.0 / self.num_micro, hidden=out)
            return inp, loss, loss.detach() / self.num_micro
        return inp, out, None

    @staticmethod
    def _backward(inp, out, grad):
        if grad is None:
            out.backward()         # last stage: `out` is the loss (gradients already carry 1/num_micro)
        else:
            out.backward(grad)
        return None if inp is None else inp.grad

    # ---- single-micro-batch steps under the reference's names (src/distributed/pipeline_scheduler.py:105-172):
    # forward_step queues (input, output); backward_step consumes the oldest pair -------------------------------
    def forward_step(self, model, input_tensor: torch.Tensor, labels: Optional[torch.Tensor] = None) -> torch.Tensor:
        """First stage: ``input_tensor`` is ``[mbs, S]`` token ids; later stages: the received activations
        ``[mbs*S(/tp), H]`` (``labels`` then gives the micro-batch shape on every stage; the last stage needs them
        for the loss).  Returns what ``send_forward`` sends on (the scaled loss on the last stage)."""
        assert labels is not None or self.pp.is_first_stage, "labels give the micro-batch shape on later stages"
        shape_src = labels if labels is not None else input_tensor
        saved, self.model = self.model, model
        try:
            if self.pp.is_first_stage:
                inp, out, _ = self._forward(input_tensor, shape_src, None)
            else:
                inp, out, _ = self._forward(None, shape_src, input_tensor)
        finally:
            self.model = saved
        self._fifo.append((inp, out))
        return out

    def backward_step(self, grad_output: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        """Backward of the oldest queued micro-batch; ``grad_output`` is ``None`` on the last stage.  Returns the
        gradient to send upstream (``None`` on the first stage)."""
        inp, out = self._fifo.popleft()
        return self._backward(inp, out, None if self.pp.is_last_stage else grad_output)

    def _track(self, name, cat):
        import contextlib
        if self.timeline is None:
            return contextlib.nullcontext()
        return self.timeline.track(name, cat, lane=f"stage{self.pp.pp_rank}")

    # ---- schedule ------------------------------------------------------------------------------------
    def run_1f1b_schedule(self, input_ids, labels=None):
        """Run all micro-batches of ``[B,S]`` (split along B).  Returns the mean loss on the last stage
        and zeros elsewhere; use :meth:`broadcast_loss` to share it.

        The reference's form ``run_1f1b_schedule(stage_model, data_iterator)`` (``num_micro_batches`` pairs of
        ``(input_ids, labels)``; src/distributed/pipeline_scheduler.py:174-320) is accepted too and returns what the
        reference returns: the accumulated loss on the last stage, ``None`` on the others."""
        if isinstance(input_ids, torch.nn.Module):
            self.model = input_ids
            pairs = [next(labels) for _ in range(self.num_micro)] if hasattr(labels, "__next__") else list(labels)
            assert len(pairs) == self.num_micro, "the iterator must yield num_micro_batches (input_ids, labels) pairs"
            total = self.run_1f1b_schedule(torch.cat([p[0] for p in pairs], 0), torch.cat([p[1] for p in pairs], 0))
            return total if self.pp.is_last_stage else None
        pp = self.pp
        dev = labels.device
        dtype = next(self.model.parameters()).dtype
        ids_mbs = input_ids.chunk(self.num_micro, dim=0)
        lab_mbs = labels.chunk(self.num_micro, dim=0)
        self._handshake(lab_mbs[0].numel(), dev, dtype)
        shape = self._act_shape
        prev, nxt, grp = pp.prev_rank, pp.next_rank, pp.group
        warm = min(pp.pp_size - 1 - pp.pp_rank, self.num_micro)
        steady = self.num_micro - warm
        fifo = deque()
        total = torch.zeros((), device=dev, dtype=torch.float32)
        f = 0

        def fwd(recv):
            nonlocal f, total
            with self._track(f"F{f}", "forward"):
                inp, out, l = self._forward(ids_mbs[f], lab_mbs[f], recv)
            if l is not None:
                total = total + l
            fifo.append((inp, out))
            f += 1
            return out

        ch = self._channels(shape, dtype, dev)
        act_in, act_out, grad_in, grad_out = ch
        for _ in range(warm):
            recv = act_in.wait(act_in.post_recv())
            out = fwd(recv)
            act_out.send(out.detach())
        for i in range(steady):
            # A receive is posted where its data is used, never ahead of compute it does not depend on: an NCCL
            # receive is a kernel that sits on the GPU until its sender arrives, and with more streams than hardware
            # queues it can hold back this rank's own compute, whose result the peer is waiting for in turn (two
            # stages that each posted a receive early stopped each other this way).  Sends are the asynchronous half:
            # a pending send only waits for the peer's host to reach its receive.
            recv = act_in.wait(act_in.post_recv())
            out = fwd(recv)
            if not pp.is_last_stage:
                act_out.send(out.detach())
            grad = grad_in.wait(grad_in.post_recv())
            inp, o = fifo.popleft()
            with self._track(f"B{i}", "backward"):
                gin = self._backward(inp, o, grad)
            if gin is not None:
                grad_out.send(gin)
        for _ in range(warm):
            grad = grad_in.wait(grad_in.post_recv())
            inp, o = fifo.popleft()
            with self._track("Bc", "backward"):
                gin = self._backward(inp, o, grad)
            if gin is not None:
                grad_out.send(gin)
        for c in ch:
            c.flush()
        return total

    def _channels(self, shape, dtype, dev):
        """(activations in, activations out, gradients in, gradients out) of this stage, built once per activation
        shape.  Activations and gradients use a communicator each (``ParallelContext.pp_fwd_group`` /
        ``pp_bwd_group``; the plain pipeline group when the context has none)."""
        key = (tuple(shape), dtype, str(dev))
        if getattr(self, "_ch_key", None) != key:
            pp = self.pp
            gf = getattr(pp.ctx, "pp_fwd_group", None) or pp.group
            gb = getattr(pp.ctx, "pp_bwd_group", None) or pp.group
            depth = pp.pp_size + 2          # received activations stay alive until their backward, plus one in flight
            self._ch = (comm.PipeChannel(gf, pp.prev_rank, shape, dtype, dev, depth),
                        comm.PipeChannel(gf, pp.next_rank, shape, dtype, dev, 0),
                        comm.PipeChannel(gb, pp.next_rank, shape, dtype, dev, 3),
                        comm.PipeChannel(gb, pp.prev_rank, shape, dtype, dev, 0))
            self._ch_key = key
        return self._ch

    def broadcast_loss(self, loss: torch.Tensor) -> torch.Tensor:
        """Share the last stage's loss with every stage of this pipeline."""
        if self.pp.pp_size > 1 and self.pp.group is not None:
            loss = loss.clone()
            dist.broadcast(loss, src=self.pp.ctx.pp_ranks[-1], group=self.pp.group)
        return loss
