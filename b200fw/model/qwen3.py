"""Qwen3-style decoder built from tensor-parallel layers.

Class names and sharding follow the reference (src/distributed/tensor_parallel.py:64-944):
``ColumnParallelLinear`` holds ``[out/tp, in]``, ``RowParallelLinear`` holds ``[out, in/tp]``,
``ParallelAttention`` does GQA with per-head QK-RMSNorm and RoPE, ``ParallelMLP`` is SwiGLU, the model
is pipeline-stage aware (embedding on the first stage, final norm + LM head on the last).

What is different by design:

* activations are token-major 2-D tensors ``[tokens, features]`` end to end;
* q/k/v and gate/up are stored fused (one GEMM each) and mapped to the HF names on load / save;
* with ``sequence_parallel`` the residual stream between blocks is sharded over the TP group along
  the token dimension, so a column layer is all-gather -> GEMM and a row layer is GEMM ->
  reduce-scatter (the reference keeps activations replicated and all-reduces);
* the residual add rides in the GEMM epilogue; norms / RoPE / SwiGLU / attention / loss are the
  kernels in :mod:`b200fw.ops`.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn as nn
import torch.utils.checkpoint

from .. import ops
from ..dist import comm
from ..dist.context import ParallelContext
from ..ops.attention import fused_qkv_attention
from .config import ModelConfig


def _tp(ctx: Optional[ParallelContext]) -> Tuple[int, int, object]:
    if ctx is None:
        return 1, 0, None
    return ctx.tp_size, ctx.tp_rank, ctx.tp_group


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-6, dtype=None, device=None):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim, dtype=dtype, device=device))

    def forward(self, x):
        shape = x.shape
        return ops.rmsnorm(x.reshape(-1, shape[-1]), self.weight, self.eps).reshape(shape)


class ColumnParallelLinear(nn.Module):
    """``y_local = x @ W_local^T`` with ``W_local = W[rank*out/tp : (rank+1)*out/tp]``.

    ``sequence_parallel``: the input is the local token shard; it is all-gathered over the TP group
    first (backward: reduce-scatter of the input gradient).  Otherwise the input is replicated and
    the backward all-reduces the input gradient.  ``gather_output`` all-gathers the last dim.
    """

    def __init__(self, in_features, out_features, ctx=None, gather_output=False, sequence_parallel=False,
                 init_std=0.02, dtype=None, device=None, bias=False):
        super().__init__()
        self.tp_size, self.tp_rank, self.tp_group = _tp(ctx)
        assert out_features % self.tp_size == 0
        # the model's projections carry no bias; the option is for layers used on their own
        # (src/distributed/tensor_parallel.py:60-118 has it): the bias is sharded with the output features
        self.bias = nn.Parameter(torch.zeros(out_features // self.tp_size, dtype=dtype, device=device)) if bias else None
        self.in_features, self.out_features = in_features, out_features
        self.out_local = out_features // self.tp_size
        self.gather_output, self.sequence_parallel = gather_output, sequence_parallel
        self.fused_comm = False     # set by the model: run the collective inside the GEMM kernel
        self.weight = nn.Parameter(torch.empty(self.out_local, in_features, dtype=dtype, device=device))
        nn.init.normal_(self.weight, std=init_std)

    def forward(self, x):
        shape = x.shape
        x = x.reshape(-1, shape[-1])
        if (self.tp_size > 1 and self.sequence_parallel and self.fused_comm and x.is_cuda and x.shape[0] % 128 == 0
                and self.bias is None):
            from ..ops import fused_tp
            y = fused_tp.column_linear_sp(x, self.weight, self.tp_group,    # all-gather inside the GEMM
                                          slot=getattr(self, "fused_slot", None))
            return y
        if self.tp_size > 1:
            x = comm.gather_sequence(x, self.tp_group) if self.sequence_parallel \
                else comm.copy_to_parallel_region(x, self.tp_group)
        y = ops.linear(x, self.weight)
        if self.bias is not None:
            y = y + self.bias
        if self.gather_output and self.tp_size > 1:
            y = comm.gather_from_parallel_region(y, self.tp_group)
        if not self.sequence_parallel:
            y = y.reshape(*shape[:-1], y.shape[-1])
        return y


class RowParallelLinear(nn.Module):
    """``y = sum_ranks x_local @ W_local^T`` with ``W_local = W[:, rank*in/tp : (rank+1)*in/tp]``.

    ``sequence_parallel``: the partial sums are reduce-scattered along tokens (the residual, already
    a token shard, is added afterwards); otherwise they are all-reduced and the residual is added on
    every rank after the reduction (so each rank keeps the full gradient of the residual stream).
    Without TP the residual add rides in the GEMM epilogue."""

    def __init__(self, in_features, out_features, ctx=None, sequence_parallel=False, init_std=0.02,
                 dtype=None, device=None, bias=False, input_is_parallel=True):
        super().__init__()
        self.tp_size, self.tp_rank, self.tp_group = _tp(ctx)
        assert in_features % self.tp_size == 0
        # bias: replicated, added once after the reduction; input_is_parallel=False: the input carries all
        # features and this rank takes its slice of the last dim (src/distributed/tensor_parallel.py:121-190)
        self.bias = nn.Parameter(torch.zeros(out_features, dtype=dtype, device=device)) if bias else None
        self.input_is_parallel = input_is_parallel
        self.in_features, self.out_features = in_features, out_features
        self.in_local = in_features // self.tp_size
        self.sequence_parallel = sequence_parallel
        self.fused_comm = False
        self.weight = nn.Parameter(torch.empty(out_features, self.in_local, dtype=dtype, device=device))
        nn.init.normal_(self.weight, std=init_std)

    def forward(self, x, residual=None):
        if not self.input_is_parallel and self.tp_size > 1:
            x = comm.scatter_to_parallel_region(x, self.tp_group)
        shape = x.shape
        x = x.reshape(-1, shape[-1])
        if self.bias is not None:
            y = self._forward_plain(x, residual) + self.bias
            return y if self.sequence_parallel else y.reshape(*shape[:-1], y.shape[-1])
        if self.tp_size == 1:
            y = ops.linear(x, self.weight, residual)
        elif self.sequence_parallel and self.fused_comm and x.is_cuda and (x.shape[0] // self.tp_size) % 128 == 0:
            from ..ops import fused_tp
            return fused_tp.row_linear_sp(x, self.weight, residual, self.tp_group)   # reduce-scatter inside the GEMM
        elif self.sequence_parallel:
            y = comm.reduce_scatter_sequence(ops.linear(x, self.weight), self.tp_group)
            if residual is not None:
                y = y + residual
        else:
            y = comm.reduce_from_parallel_region(ops.linear(x, self.weight), self.tp_group)
            if residual is not None:
                y = y + residual.reshape(y.shape)
        if not self.sequence_parallel:
            y = y.reshape(*shape[:-1], y.shape[-1])
        return y


def _row_forward_plain(self, x, residual=None):
    """Library-collective form of the row-parallel product on 2-D ``x`` (no fused kernel, no epilogue add)."""
    y = ops.linear(x, self.weight)
    if self.tp_size > 1:
        y = comm.reduce_scatter_sequence(y, self.tp_group) if self.sequence_parallel \
            else comm.reduce_from_parallel_region(y, self.tp_group)
    return y if residual is None else y + residual.reshape(y.shape)


RowParallelLinear._forward_plain = _row_forward_plain


class _ProjectionView:
    """Half of a fused projection under the name a separate layer would have (``mlp.gate_proj.weight``)."""

    def __init__(self, fused: ColumnParallelLinear, half: int):
        self._fused, self._half = fused, half

    @property
    def weight(self) -> torch.Tensor:
        n = self._fused.out_local // 2
        return self._fused.weight[self._half * n:(self._half + 1) * n]


class ParallelMLP(nn.Module):
    """SwiGLU FFN; gate and up projections are one fused column-parallel GEMM ([gate_local | up_local])."""

    def __init__(self, cfg, ctx=None, sequence_parallel=False, dtype=None, device=None):
        """``ParallelMLP(model_config, ctx, ...)``; the reference's ``ParallelMLP(hidden_size, intermediate_size, ctx)``
        (src/distributed/tensor_parallel.py:300-340) is accepted as well."""
        super().__init__()
        if isinstance(cfg, int):
            from types import SimpleNamespace
            hidden, inter = cfg, ctx
            ctx = None if isinstance(sequence_parallel, bool) else sequence_parallel
            sequence_parallel = False
            cfg = SimpleNamespace(hidden_size=hidden, intermediate_size=inter, init_std=0.02)
        self.sequence_parallel = sequence_parallel
        self.gate_up_proj = ColumnParallelLinear(cfg.hidden_size, 2 * cfg.intermediate_size, ctx,
                                                 sequence_parallel=sequence_parallel, init_std=cfg.init_std,
                                                 dtype=dtype, device=device)
        self.down_proj = RowParallelLinear(cfg.intermediate_size, cfg.hidden_size, ctx,
                                           sequence_parallel=sequence_parallel, init_std=cfg.init_std,
                                           dtype=dtype, device=device)

    @property
    def gate_proj(self) -> _ProjectionView:
        return _ProjectionView(self.gate_up_proj, 0)

    @property
    def up_proj(self) -> _ProjectionView:
        return _ProjectionView(self.gate_up_proj, 1)

    def forward(self, x, residual=None):
        gu = self.gate_up_proj(x)
        y = self.down_proj(ops.swiglu(gu.reshape(-1, gu.shape[-1])), residual)
        if x.dim() > 2 and y.dim() == 2 and not self.sequence_parallel:
            y = y.reshape(*x.shape[:-1], y.shape[-1])
        return y


class ParallelAttention(nn.Module):
    """Causal GQA attention; q/k/v are one fused column-parallel GEMM ([q_local | k_local | v_local]),
    q and k get per-head RMSNorm and half-rotation RoPE."""

    def __init__(self, cfg: ModelConfig, ctx=None, sequence_parallel=False, dtype=None, device=None):
        super().__init__()
        tp, _, _ = _tp(ctx)
        assert cfg.num_heads % tp == 0 and cfg.num_kv_heads % tp == 0, "heads must divide by tp"
        self.cfg = cfg
        self.heads_local, self.kv_heads_local = cfg.num_heads // tp, cfg.num_kv_heads // tp
        D = cfg.head_dim
        self.qkv_proj = ColumnParallelLinear(cfg.hidden_size, (cfg.num_heads + 2 * cfg.num_kv_heads) * D, ctx,
                                             sequence_parallel=sequence_parallel, init_std=cfg.init_std,
                                             dtype=dtype, device=device)
        self.o_proj = RowParallelLinear(cfg.num_heads * D, cfg.hidden_size, ctx,
                                        sequence_parallel=sequence_parallel, init_std=cfg.init_std,
                                        dtype=dtype, device=device)
        self.q_norm = RMSNorm(D, cfg.rms_norm_eps, dtype=dtype, device=device)
        self.k_norm = RMSNorm(D, cfg.rms_norm_eps, dtype=dtype, device=device)

    def forward(self, x, positions, B, S, residual=None):
        cfg = self.cfg
        qkv = self.qkv_proj(x)
        qkv = qkv.reshape(-1, qkv.shape[-1])
        cos, sin = ops.rope_tables(cfg.max_position_embeddings, cfg.head_dim, cfg.rope_theta, qkv.device)
        att = fused_qkv_attention(qkv, self.q_norm.weight, self.k_norm.weight, positions, cos, sin, B, S,
                                  self.heads_local, self.kv_heads_local, cfg.head_dim, cfg.rms_norm_eps)
        return self.o_proj(att, residual)


class ParallelTransformerLayer(nn.Module):
    def __init__(self, cfg: ModelConfig, ctx=None, sequence_parallel=False, dtype=None, device=None):
        super().__init__()
        self.input_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype=dtype, device=device)
        self.self_attn = ParallelAttention(cfg, ctx, sequence_parallel, dtype=dtype, device=device)
        self.post_attention_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype=dtype, device=device)
        self.mlp = ParallelMLP(cfg, ctx, sequence_parallel, dtype=dtype, device=device)

    def forward(self, h, positions, B, S):
        h = self.self_attn(self.input_layernorm(h), positions, B, S, residual=h)
        h = self.mlp(self.post_attention_layernorm(h), residual=h)
        return h


class ParallelTransformerModel(nn.Module):
    """Decoder stack for one pipeline stage.

    ``layer_range`` = (start, end) global layer indices owned by this stage (default: all); the
    embedding lives on the first stage, final norm + LM head on the last.  Weight tying is only
    possible when one stage holds both (src/distributed/tensor_parallel.py:784-851).
    """

    def __init__(self, cfg: Optional[ModelConfig] = None, ctx: Optional[ParallelContext] = None,
                 layer_range: Optional[Tuple[int, int]] = None, is_first_stage: bool = True,
                 is_last_stage: bool = True, sequence_parallel: bool = False,
                 gradient_checkpointing: bool = False, dtype=None, device=None,
                 vocab_parallel: bool = True, **reference_kwargs):
        super().__init__()
        if cfg is None or reference_kwargs:
            # the reference's keyword form (src/distributed/tensor_parallel.py:750-770): the architecture spelled out
            # field by field, ``parallel_context`` and an optional ``pp_context`` that selects this stage's layers
            kw = dict(reference_kwargs)
            ctx = kw.pop("parallel_context", ctx)
            ppc = kw.pop("pp_context", None)
            gradient_checkpointing = bool(kw.pop("use_gradient_checkpoint", gradient_checkpointing))
            for ignored in ("use_flash_attn", "enable_comm_overlap", "stream_manager", "attention_backend"):
                kw.pop(ignored, None)           # attention is always the native kernel; overlap needs no switch here
            if cfg is None:
                kw.setdefault("tie_word_embeddings", False)
                cfg = ModelConfig(**kw)
            elif kw:
                raise TypeError(f"unexpected arguments: {sorted(kw)}")
            if ppc is not None and ppc.pp_size > 1:
                layer_range = (ppc.layer_start, ppc.layer_end)
                is_first_stage, is_last_stage = ppc.is_first_stage, ppc.is_last_stage
            if ctx is not None and not hasattr(ctx, "tp_rank"):
                ctx = None
        self.cfg, self.ctx = cfg, ctx
        self.tp_size, self.tp_rank, self.tp_group = _tp(ctx)
        self.sequence_parallel = sequence_parallel and self.tp_size > 1
        self.gradient_checkpointing = gradient_checkpointing
        self.layer_start, self.layer_end = layer_range if layer_range is not None else (0, cfg.num_layers)
        self.is_first_stage, self.is_last_stage = is_first_stage, is_last_stage
        self.compact_ignored_rows = True   # LM head runs on rows with a real label only (exact)
        self.embed_tokens = None
        if is_first_stage:
            self.embed_tokens = nn.Parameter(torch.empty(cfg.vocab_size, cfg.hidden_size, dtype=dtype, device=device))
            nn.init.normal_(self.embed_tokens, std=cfg.init_std)
        self.layers = nn.ModuleList([
            ParallelTransformerLayer(cfg, ctx, self.sequence_parallel, dtype=dtype, device=device)
            for _ in range(self.layer_start, self.layer_end)])
        self.norm = None
        self.lm_head = None
        self.tied = False
        # An untied LM head is sharded over the vocabulary across the TP group (each rank computes its
        # slice of the logits; the losses exchange three floats per token).  A tied head stays
        # replicated with the embedding, as the reference keeps both (tensor_parallel.py:784-851).
        self.vocab_parallel = bool(vocab_parallel and is_last_stage and self.tp_size > 1
                                   and not (cfg.tie_word_embeddings and is_first_stage)
                                   and cfg.vocab_size % (8 * self.tp_size) == 0)
        if is_last_stage:
            self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype=dtype, device=device)
            self.tied = cfg.tie_word_embeddings and is_first_stage
            if not self.tied:
                rows = cfg.vocab_size // self.tp_size if self.vocab_parallel else cfg.vocab_size
                self.lm_head = nn.Parameter(torch.empty(rows, cfg.hidden_size, dtype=dtype, device=device))
                nn.init.normal_(self.lm_head, std=cfg.init_std)
        self._tag_parameters()

    def set_fused_comm(self, on: bool = True):
        """Run every sequence-parallel linear's collective inside its GEMM kernel (peer loads / stores
        over NVLink) instead of as separate NCCL calls."""
        import re
        for name, m in self.named_modules():
            if isinstance(m, (ColumnParallelLinear, RowParallelLinear)):
                m.fused_comm = on and self.sequence_parallel
                # gather-buffer slot of a column-parallel layer: its gathered input is saved for the weight gradient.
                # With gradient checkpointing a layer's forward is recomputed right before its backward, so one slot
                # per role serves all layers; without it every layer keeps its own until the backward pass.
                role = [p for p in name.split(".") if p.endswith("_proj")]
                li = re.search(r"layers\.(\d+)\.", name)
                m.fused_slot = (role[0] if role else name,
                                -1 if (self.gradient_checkpointing or li is None) else int(li.group(1)))

    def _tag_parameters(self):
        # parameters whose per-rank gradient is only a partial sum under TP (their inputs are head-
        # or token-sharded): they need a SUM over the TP group.  Everything else replicated already
        # sees the full gradient on every rank.
        for name, p in self.named_parameters():
            p.tp_partial_grad = self.tp_size > 1 and (
                "q_norm" in name or "k_norm" in name or
                (self.sequence_parallel and ("layernorm" in name or name == "norm.weight")))
            p.tp_sharded = self.tp_size > 1 and (
                "qkv_proj" in name or "gate_up_proj" in name or "o_proj" in name or "down_proj" in name
                or (name == "lm_head" and self.vocab_parallel))
        if self.tied and self.embed_tokens is not None:
            self.embed_tokens.grad_contribs = 2  # LM head (in the loss) and embedding both write its gradient

    @torch.no_grad()
    def init_weights(self, seed: int = 0, std: Optional[float] = None):
        """Deterministic N(0, std) init that is identical on every data-parallel rank, identical across
        TP ranks for replicated parameters and distinct per TP rank for sharded ones; norm weights = 1.
        Generated on the parameter's device (no full-size CPU staging)."""
        import zlib
        std = self.cfg.init_std if std is None else std
        for name, p in self.named_parameters():
            if p.dim() == 1:
                p.fill_(1.0)
                continue
            key = zlib.crc32(f"{self.layer_start}:{name}".encode()) + 1000003 * seed
            if getattr(p, "tp_sharded", False):
                key += 7919 * (self.tp_rank + 1)
            g = torch.Generator(device=p.device).manual_seed(key % (2 ** 62))
            p.copy_(torch.empty(p.shape, dtype=torch.float32, device=p.device).normal_(0.0, std, generator=g).to(p.dtype))

    def clone(self, requires_grad: bool = False) -> "ParallelTransformerModel":
        """A second model with the same architecture, parallel layout and weights (process groups are
        shared, not copied); used for the frozen reference policy."""
        p0 = next(self.parameters())
        other = ParallelTransformerModel(self.cfg, self.ctx, (self.layer_start, self.layer_end),
                                         self.is_first_stage, self.is_last_stage, self.sequence_parallel,
                                         self.gradient_checkpointing, dtype=p0.dtype, device=p0.device,
                                         vocab_parallel=self.vocab_parallel)
        with torch.no_grad():
            for a, b in zip(other.parameters(), self.parameters()):
                a.copy_(b)
                a.requires_grad_(requires_grad)
        return other

    # ---- pieces ------------------------------------------------------------------------------
    @property
    def lm_head_weight(self) -> torch.Tensor:
        return self.embed_tokens if self.tied else self.lm_head

    def _positions(self, B: int, S: int, device, positions=None):
        if positions is not None:
            return positions.reshape(-1).to(torch.int32)
        if S > self.cfg.max_position_embeddings:
            # the rotary kernels index the cos / sin tables with the position, unchecked
            raise ValueError(f"sequence length {S} exceeds max_position_embeddings={self.cfg.max_position_embeddings}")
        return torch.arange(S, device=device, dtype=torch.int32).repeat(B)

    def embed(self, input_ids: torch.Tensor) -> torch.Tensor:
        h = ops.embedding(input_ids.reshape(-1), self.embed_tokens)
        if self.sequence_parallel:
            h = comm.scatter_to_sequence_region(h, self.tp_group)
        return h

    def run_layers(self, h: torch.Tensor, positions: torch.Tensor, B: int, S: int) -> torch.Tensor:
        for layer in self.layers:
            if self.gradient_checkpointing and torch.is_grad_enabled():
                h = torch.utils.checkpoint.checkpoint(layer, h, positions, B, S, use_reentrant=False)
            else:
                h = layer(h, positions, B, S)
        return h

    def final_hidden(self, h: torch.Tensor) -> torch.Tensor:
        """Final norm; under sequence parallelism the result is gathered to all tokens.  With a
        vocabulary-sharded head every rank's hidden-state gradient is a partial sum, so the gather's
        backward is a reduce-scatter; with a replicated head it is a plain slice."""
        h = self.norm(h)
        if self.sequence_parallel:
            h = (comm.gather_sequence if self.vocab_parallel else comm.gather_sequence_replicated)(h, self.tp_group)
        return h

    def vocab_shard(self) -> Optional[ops.VocabShard]:
        if not self.vocab_parallel:
            return None
        return ops.VocabShard(self.tp_group, self.tp_rank, self.tp_size, self.cfg.vocab_size,
                              reduce_dh=not self.sequence_parallel)

    def logits_from_hidden(self, h: torch.Tensor) -> torch.Tensor:
        """``[M,H]`` final hidden states -> ``[M,V]`` logits (all-gathered over the vocabulary shards)."""
        if not self.vocab_parallel:
            return ops.linear(h, self.lm_head_weight)
        if not self.sequence_parallel:
            h = comm.copy_to_parallel_region(h, self.tp_group)
        return comm.gather_from_parallel_region(ops.linear(h, self.lm_head), self.tp_group)

    # ---- public entry points ---------------------------------------------------------------------
    def forward_hidden(self, input_or_hidden: torch.Tensor, B: int, S: int, positions=None) -> torch.Tensor:
        """Stage forward: token ids (first stage) or the previous stage's activations ``[B*S(/tp), H]``
        in, this stage's output activations (or the final normed hidden states on the last stage) out."""
        dev = input_or_hidden.device
        pos = self._positions(B, S, dev, positions)
        h = self.embed(input_or_hidden) if self.is_first_stage else input_or_hidden
        h = self.run_layers(h, pos, B, S)
        if self.is_last_stage:
            h = self.final_hidden(h)
        return h

    def forward(self, input_ids: torch.Tensor, positions=None, attention_mask=None) -> torch.Tensor:
        """``[B,S]`` token ids -> ``[B,S,V]`` logits (materialised; the training losses use
        :meth:`loss` / :meth:`token_logprobs`, which never build this tensor).  ``attention_mask`` is
        accepted for API compatibility: attention is causal and padding sits on the right, so padded
        positions never influence real ones."""
        if input_ids.dim() == 3:
            # a later pipeline stage fed ``[B,S,H]`` activations (the reference's stage models take and return them
            # in this shape: src/distributed/tensor_parallel.py:853-905)
            assert not self.is_first_stage and not self.sequence_parallel
            B, S, H = input_ids.shape
            h = self.forward_hidden(input_ids.reshape(B * S, H), B, S, positions)
        else:
            B, S = input_ids.shape
            h = self.forward_hidden(input_ids, B, S, positions)
        if not self.is_last_stage:
            return h if self.sequence_parallel else h.reshape(B, S, -1)
        return self.logits_from_hidden(h).reshape(B, S, -1)

    @property
    def stage_start(self) -> int:
        """Global index of this stage's first layer (the reference's name)."""
        return self.layer_start

    def loss(self, input_ids: torch.Tensor, labels: torch.Tensor, loss_scale: float = 1.0,
             hidden: Optional[torch.Tensor] = None, valid_idx: Optional[torch.Tensor] = None,
             valid_labels: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Next-token CE with the shift done on the labels (``labels[:, t]`` supervises the logits at
        ``t-1``); ``-100`` is ignored.  Same value as the reference's shifted ``F.cross_entropy``
        (src/engines/train_engine.py:44-50)."""
        if valid_labels is not None:
            # static-shape form (CUDA-graph replay): row indices and their labels come padded to a fixed
            # length, padding rows carry label -100 and add nothing
            B, S = input_ids.shape
            h = hidden if hidden is not None else self.forward_hidden(input_ids, B, S)
            return ops.lm_head_cross_entropy(h.index_select(0, valid_idx), self.lm_head_weight, valid_labels,
                                             loss_scale=loss_scale, shard=self.vocab_shard())
        B, S = labels.shape
        h = hidden if hidden is not None else self.forward_hidden(input_ids, B, S)
        shifted = torch.full_like(labels, -100)
        shifted[:, :-1] = labels[:, 1:]
        shifted = shifted.reshape(-1)
        if self.compact_ignored_rows:
            # masked positions (prompt tokens, padding) add nothing to the loss or its gradient: run the
            # LM head on the supervised rows only
            # ``valid_idx``: the caller already knows the supervised rows (computed on the host)
            idx = valid_idx if valid_idx is not None else ops.valid_rows(shifted)
            if idx is not None:
                if idx.numel() == 0:
                    return h.float().sum() * 0.0
                h, shifted = h.index_select(0, idx), shifted.index_select(0, idx)
        return ops.lm_head_cross_entropy(h, self.lm_head_weight, shifted, loss_scale=loss_scale,
                                         shard=self.vocab_shard())

    def token_logprobs(self, input_ids: torch.Tensor, temperature: float = 1.0,
                       hidden: Optional[torch.Tensor] = None,
                       labels: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``[B,S-1]`` log-prob of token ``t+1`` under the logits at ``t``.  With ``labels`` only the
        positions whose label is not ``-100`` are scored (others return 0)."""
        B, S = input_ids.shape
        h = hidden if hidden is not None else self.forward_hidden(input_ids, B, S)
        src = input_ids if labels is None else labels
        tgt = torch.full_like(input_ids, -100)
        tgt[:, :-1] = src[:, 1:]
        tgt = tgt.reshape(-1)
        idx = ops.valid_rows(tgt) if (labels is not None and self.compact_ignored_rows) else None
        if idx is None:
            lp = ops.lm_head_logprob(h, self.lm_head_weight, tgt, temperature, shard=self.vocab_shard())
        else:
            lp = torch.zeros(B * S, dtype=torch.float32, device=h.device)
            if idx.numel() > 0:
                sel = ops.lm_head_logprob(h.index_select(0, idx), self.lm_head_weight, tgt.index_select(0, idx),
                                          temperature, shard=self.vocab_shard())
                lp = lp.index_copy(0, idx, sel)
            elif torch.is_grad_enabled() and h.requires_grad:
                # nothing to score on this rank (every response empty): keep the result attached to the graph so that
                # backward still runs, with zero gradients, and data-parallel peers are not left waiting for this rank
                lp = lp + h.float().sum() * 0.0
        return lp.reshape(B, S)[:, :-1]
