"""LoRA on tensor-parallel linears.

Same roles as the reference (src/distributed/lora.py:46-416): ``LoRAColumnParallel`` shards ``B`` with
the base layer's output rows and replicates ``A``; ``LoRARowParallel`` shards ``A`` with the base
layer's input columns, all-reduces the rank-r intermediate and replicates ``B``.  ``apply_lora`` freezes
the base model and attaches adapters by HF target name; because q|k|v and gate|up are stored fused, a
fused layer carries one adapter per targeted sub-projection, each writing its own column range.
Adapter parameters are fp32; the low-rank products run in the activation dtype.
"""
from __future__ import annotations

import math
import os
from typing import Dict, Iterable, List, Optional, Tuple

import torch
import torch.nn as nn

from ..dist import comm
from .qwen3 import RowParallelLinear, ParallelAttention, ParallelMLP

DEFAULT_TARGETS = ["q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj"]


class LoRALayer(nn.Module):
    """Plain (unsharded) adapter: ``delta(x) = (x A^T) B^T * alpha/r``; A kaiming-uniform, B zero."""

    def __init__(self, in_features, out_features, rank=16, alpha=32.0, device=None, dropout: float = 0.0):
        super().__init__()
        if isinstance(device, float):            # the reference's fifth argument is the dropout rate
            device, dropout = None, device
        if dropout:
            raise ValueError("LoRA dropout is not supported: use dropout=0")
        self.rank, self.alpha, self.scaling = rank, alpha, alpha / rank
        self.lora_A = nn.Parameter(torch.empty(rank, in_features, dtype=torch.float32, device=device))
        self.lora_B = nn.Parameter(torch.zeros(out_features, rank, dtype=torch.float32, device=device))
        nn.init.kaiming_uniform_(self.lora_A, a=math.sqrt(5))

    def delta(self, x):
        a = self.lora_A.to(x.dtype)
        b = self.lora_B.to(x.dtype)
        return (x @ a.t()) @ b.t() * self.scaling

    def forward(self, x):
        return self.delta(x)

    def delta_weight(self) -> torch.Tensor:
        return (self.lora_B @ self.lora_A) * self.scaling


class LoRAColumnParallel(LoRALayer):
    """A ``[r, in]`` replicated (its gradient is a partial sum over TP ranks), B ``[out/tp, r]`` sharded."""

    def __init__(self, in_features, out_local, rank, alpha, tp_group=None, device=None):
        super().__init__(in_features, out_local, rank, alpha, device)
        self.tp_group = tp_group
        self.lora_A.tp_partial_grad = tp_group is not None
        self.lora_B.tp_sharded = tp_group is not None


class LoRARowParallel(LoRALayer):
    """A ``[r, in/tp]`` sharded, B ``[out, r]`` replicated; the rank-r intermediate is all-reduced
    (reduce-scattered over the sequence under sequence parallelism)."""

    def __init__(self, in_local, out_features, rank, alpha, tp_group=None, device=None,
                 sequence_parallel: bool = False):
        super().__init__(in_local, out_features, rank, alpha, device)
        self.tp_group = tp_group
        self.lora_A.tp_sharded = tp_group is not None
        # after a plain all-reduce every rank sees the full gradient of B; under sequence parallelism
        # each rank only sees its own tokens' contribution
        self.lora_B.tp_partial_grad = tp_group is not None and sequence_parallel

    def delta(self, x):
        a = self.lora_A.to(x.dtype)
        b = self.lora_B.to(x.dtype)
        mid = x @ a.t()
        mid = comm.reduce_from_parallel_region(mid, self.tp_group)
        return mid @ b.t() * self.scaling


class LinearWithLoRA(nn.Module):
    """Wraps a (possibly fused) parallel linear; ``adapters`` maps a target name to
    ``(adapter, col_start, col_end)`` in the wrapped layer's local output columns."""

    def __init__(self, base: nn.Module, adapters: Dict[str, Tuple[LoRALayer, int, int]]):
        super().__init__()
        self.base = base
        self.adapters = nn.ModuleDict({k: v[0] for k, v in adapters.items()})
        self.ranges = {k: (v[1], v[2]) for k, v in adapters.items()}
        self.merged = False
        # False (or B200FW_LORA_FUSE=0): base projection, then two adapter GEMMs (the only form under TP)
        self.fuse_into_base = os.environ.get("B200FW_LORA_FUSE", "1") != "0"
        self._plan_cache = None
        if getattr(base, "tp_size", 1) == 1 and self.fuse_into_base and base.weight.dtype == torch.bfloat16:
            # the fused op writes these parameters' gradients itself (into the optimizer's bucket views when it has
            # them): an optimizer may bind ``main_grad`` buffers to them as it does for bf16 weights
            for ad in self.adapters.values():
                ad.lora_A.direct_grad = True
                ad.lora_B.direct_grad = True

    @property
    def weight(self):
        return self.base.weight

    @torch.no_grad()
    def merged_weight(self) -> torch.Tensor:
        """A new tensor ``W + sum_i scaling_i * B_i A_i`` (shard-local under TP); the frozen base weight is not
        touched, as in the reference's export (src/distributed/lora.py:385-391).  A bf16 ``(W + d) - d`` does
        not give back ``W`` bit for bit, so merging in place and undoing it would move the base a little on
        every export."""
        w = self.base.weight.detach().clone()
        if self.merged:
            return w
        row = isinstance(self.base, RowParallelLinear)
        for name, ad in self.adapters.items():
            dw = ad.delta_weight().to(w.dtype)
            if row:
                w.add_(dw)
            else:
                s, e = self.ranges[name]
                w[s:e].add_(dw)
        return w

    def _stacked(self, dtype):
        """All adapters of this layer as one pair: ``A_cat [R, in]`` (adapters stacked along the rank
        dimension) and ``B_bd [out_local, R]`` (each adapter's B, times its scaling, in its own row range
        and rank columns; zero elsewhere), so the layer's whole LoRA update is two GEMMs."""
        order = sorted(self.ranges.items(), key=lambda kv: kv[1][0])
        ads = [self.adapters[name] for name, _ in order]
        if len(ads) == 1 and order[0][1] == (0, self.base.weight.shape[0]):
            return ads[0].lora_A.to(dtype), (ads[0].lora_B * ads[0].scaling).to(dtype)
        a_cat = torch.cat([ad.lora_A for ad in ads], 0).to(dtype)
        b_bd = torch.zeros(self.base.weight.shape[0], a_cat.shape[0], dtype=dtype, device=a_cat.device)
        r0 = 0
        for ad, (_, (s0, e0)) in zip(ads, order):
            b_bd[s0:e0, r0:r0 + ad.rank] = (ad.lora_B * ad.scaling).to(dtype)
            r0 += ad.rank
        return a_cat, b_bd

    def _total_rank(self) -> int:
        return sum(ad.rank for ad in self.adapters.values())

    def _grad_plan(self):
        """``(rank offset, rank, first row, last row, scaling)`` per adapter in the stacking order of ``_stacked``, and
        the adapters' parameters ``A_0, B_0, A_1, B_1, ...``: how the fused op hands the stacked gradients back."""
        if self._plan_cache is None:
            order = sorted(self.ranges.items(), key=lambda kv: kv[1][0])
            plan, params, r0 = [], [], 0
            for name, (s0, e0) in order:
                ad = self.adapters[name]
                plan.append((r0, ad.rank, s0, e0, float(ad.scaling)))
                params += [ad.lora_A, ad.lora_B]
                r0 += ad.rank
            self._plan_cache = (tuple(plan), tuple(params))
        return self._plan_cache

    def forward(self, x, residual=None):
        from .. import ops
        base = self.base
        is_row = isinstance(base, RowParallelLinear)
        if self.merged or not self.adapters:
            return base(x, residual) if is_row else base(x)
        tp, grp, sp = base.tp_size, base.tp_group, base.sequence_parallel
        x2 = x.reshape(-1, x.shape[-1])
        fused = (self.fuse_into_base and tp == 1 and x2.is_cuda and base.bias is None and self._total_rank() % 8 == 0
                 and x2.dtype == torch.bfloat16)
        with torch.set_grad_enabled(torch.is_grad_enabled() and not fused):
            a_cat, b_bd = self._stacked(x2.dtype)        # fused: no autograd graph through the stacking
        if fused:
            # one device: the rank-R update rides in the base projection's GEMM (forward and input gradient), the
            # frozen base weight gets no gradient GEMM at all
            plan, params = self._grad_plan()
            y = ops.lora_linear(x2 if x2.is_contiguous() else x2.contiguous(), base.weight, a_cat.contiguous(), b_bd,
                                residual.reshape(-1, base.weight.shape[0]) if residual is not None else None,
                                plan=plan, params=params)
            return y.reshape(*x.shape[:-1], y.shape[-1])
        y = base(x, residual) if is_row else base(x)
        if is_row:
            # x holds this rank's input columns: the rank-R intermediate is a partial sum over TP
            mid = ops.linear(x2, a_cat)
            if tp > 1:
                mid = comm.reduce_scatter_sequence(mid, grp) if sp else comm.reduce_from_parallel_region(mid, grp)
        else:
            if tp > 1 and not sp:
                x2 = comm.copy_to_parallel_region(x2, grp)
            mid = ops.linear(x2, a_cat)
            if tp > 1 and sp:
                mid = comm.gather_sequence(mid, grp)   # [tokens/tp, R] -> [tokens, R]: R columns, not hidden
        shape = y.shape
        return ops.linear(mid, b_bd, residual=y.reshape(-1, shape[-1])).reshape(shape)


def _sub_ranges(parent) -> Dict[str, Tuple[str, int, int]]:
    """target name -> (attribute of the fused layer on ``parent``, local col start, local col end)."""
    out = {}
    if isinstance(parent, ParallelAttention):
        D = parent.cfg.head_dim
        hq, hk = parent.heads_local * D, parent.kv_heads_local * D
        out["q_proj"] = ("qkv_proj", 0, hq)
        out["k_proj"] = ("qkv_proj", hq, hq + hk)
        out["v_proj"] = ("qkv_proj", hq + hk, hq + 2 * hk)
        out["o_proj"] = ("o_proj", 0, parent.o_proj.out_features)
    elif isinstance(parent, ParallelMLP):
        base = parent.gate_up_proj.base if isinstance(parent.gate_up_proj, LinearWithLoRA) else parent.gate_up_proj
        il = base.out_local // 2
        out["gate_proj"] = ("gate_up_proj", 0, il)
        out["up_proj"] = ("gate_up_proj", il, 2 * il)
        out["down_proj"] = ("down_proj", 0, parent.down_proj.out_features)
    return out


def apply_lora(model: nn.Module, rank=16, alpha=32.0, target_modules: Optional[Iterable[str]] = None):
    """Freeze every existing parameter and attach adapters to the targeted projections.
    Returns the qualified names of the adapted sub-projections.

    The reference's call ``apply_lora(model, lora_config, parallel_context)`` (src/distributed/lora.py:259-343: a dict
    with ``rank`` / ``alpha`` / ``target_modules`` / ``dropout``) is recognised by the dict in second place and returns
    the model, as the reference does; the names are then in ``model.lora_adapted_names``.  (The parallel layout is
    read from the layers themselves; adapter dropout is not implemented and a non-zero value is refused.)"""
    if isinstance(rank, dict):
        cfg = rank
        if float(cfg.get("dropout", 0.0) or 0.0) != 0.0:
            raise ValueError("LoRA dropout is not supported: set lora.dropout to 0")
        names = apply_lora(model, int(cfg.get("rank", 16)), float(cfg.get("alpha", 32.0)),
                           cfg.get("target_modules") or None)
        model.lora_adapted_names = names
        return model
    targets = list(target_modules) if target_modules is not None else list(DEFAULT_TARGETS)
    for p in model.parameters():
        p.requires_grad_(False)
    adapted: List[str] = []
    for mod_name, parent in list(model.named_modules()):
        table = _sub_ranges(parent)
        if not table:
            continue
        per_attr: Dict[str, Dict[str, Tuple[LoRALayer, int, int]]] = {}
        for tgt in targets:
            if tgt not in table:
                continue
            attr, s, e = table[tgt]
            base = getattr(parent, attr)
            if isinstance(base, LinearWithLoRA):
                continue
            dev = base.weight.device
            grp = base.tp_group if base.tp_size > 1 else None
            if isinstance(base, RowParallelLinear):
                ad = LoRARowParallel(base.in_local, base.out_features, rank, alpha, grp, dev,
                                     sequence_parallel=base.sequence_parallel)
            else:
                ad = LoRAColumnParallel(base.in_features, e - s, rank, alpha, grp, dev)
            per_attr.setdefault(attr, {})[tgt] = (ad, s, e)
            adapted.append(f"{mod_name}.{tgt}")
        for attr, ads in per_attr.items():
            setattr(parent, attr, LinearWithLoRA(getattr(parent, attr), ads))
    return adapted


def iter_lora(model: nn.Module):
    for name, mod in model.named_modules():
        if isinstance(mod, LinearWithLoRA):
            for tgt, ad in mod.adapters.items():
                yield name, tgt, mod, ad


@torch.no_grad()
def merge_lora_weights(model: nn.Module, unmerge: bool = False) -> int:
    """``W += scaling * B A`` on the targeted row / column ranges (``unmerge`` subtracts).  Works
    shard-locally under TP: column adapters hold the matching rows of B, row adapters the matching
    columns of A."""
    n = 0
    sign = -1.0 if unmerge else 1.0
    for _, tgt, mod, ad in iter_lora(model):
        s, e = mod.ranges[tgt]
        w = mod.base.weight
        dw = ad.delta_weight().to(w.dtype)
        if isinstance(mod.base, RowParallelLinear):
            w.add_(dw, alpha=sign)
        else:
            w[s:e].add_(dw, alpha=sign)
        n += 1
    for m in model.modules():
        if isinstance(m, LinearWithLoRA):
            m.merged = not unmerge
    return n


def get_lora_state_dict(model: nn.Module) -> Dict[str, torch.Tensor]:
    """``{qualified.target.lora_A|lora_B: tensor}`` of this rank's adapter shards."""
    out = {}
    for name, tgt, _, ad in iter_lora(model):
        out[f"{name}.{tgt}.lora_A"] = ad.lora_A.detach()
        out[f"{name}.{tgt}.lora_B"] = ad.lora_B.detach()
    return out


@torch.no_grad()
def flat_lora_state(model: nn.Module):
    """The same content as :func:`get_lora_state_dict` as a :class:`b200fw.sync.double_buffer.FlatState`: one fp32
    tensor holding a COPY of every adapter tensor back to back (one concatenation), with the named tensors as views
    on demand.  The layout is computed once per model."""
    from ..sync.double_buffer import FlatLayout, FlatState
    cache = model.__dict__.get("_flat_lora_cache")
    if cache is None:
        keys, params = [], []
        for name, tgt, _, ad in iter_lora(model):
            keys += [f"{name}.{tgt}.lora_A", f"{name}.{tgt}.lora_B"]
            params += [ad.lora_A, ad.lora_B]
        cache = model.__dict__["_flat_lora_cache"] = (FlatLayout(keys, [p.shape for p in params]), params)
    layout, params = cache
    return FlatState(layout, torch.cat([p.detach().reshape(-1).float() for p in params]))


@torch.no_grad()
def load_lora_state_dict(model: nn.Module, state: Dict[str, torch.Tensor]) -> int:
    n = 0
    for name, tgt, _, ad in iter_lora(model):
        for leaf in ("lora_A", "lora_B"):
            key = f"{name}.{tgt}.{leaf}"
            if key in state:
                getattr(ad, leaf).copy_(state[key].to(getattr(ad, leaf).dtype))
                n += 1
    return n
