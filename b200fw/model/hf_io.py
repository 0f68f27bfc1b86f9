"""HF-style checkpoint IO and the tensor-parallel shard rule.

Layout contract (the reference's loader, src/distributed/tensor_parallel.py:952-1064): a directory
with ``config.json`` and ``*.safetensors`` (or ``pytorch_model.bin``) whose keys are
``model.embed_tokens.weight``, ``model.layers.N.self_attn.{q,k,v,o}_proj.weight``,
``model.layers.N.self_attn.{q,k}_norm.weight``, ``model.layers.N.mlp.{gate,up,down}_proj.weight``,
``model.layers.N.{input,post_attention}_layernorm.weight``, ``model.norm.weight``, ``lm_head.weight``.
q/k/v/gate/up are sliced on dim 0 per TP rank, o/down on dim 1, everything else is replicated;
local layer ``i`` of a pipeline stage maps to global layer ``layer_start + i``.  This framework keeps
q|k|v and gate|up fused in memory; the functions here fuse on load and split on save, so files on
disk always carry the plain HF names.  Saving exists because the reference never writes base weights
back, which makes full-SFT results unrecoverable.
"""
from __future__ import annotations

import glob
import json
import os
from typing import Dict, Iterator, Tuple

import torch

from .config import ModelConfig


def read_hf_config(path: str) -> ModelConfig:
    with open(os.path.join(path, "config.json")) as f:
        return ModelConfig.from_hf(json.load(f))


def write_hf_config(path: str, cfg: ModelConfig) -> None:
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg.to_hf(), f, indent=2)


def _load_all(path: str) -> Dict[str, torch.Tensor]:
    tensors: Dict[str, torch.Tensor] = {}
    files = sorted(glob.glob(os.path.join(path, "*.safetensors")))
    if files:
        from safetensors.torch import load_file
        for f in files:
            tensors.update(load_file(f, device="cpu"))
        return tensors
    binf = os.path.join(path, "pytorch_model.bin")
    if os.path.exists(binf):
        return torch.load(binf, map_location="cpu", weights_only=True)
    return tensors


def _rows(t: torch.Tensor, rank: int, tp: int) -> torch.Tensor:
    n = t.shape[0] // tp
    return t[rank * n:(rank + 1) * n]


def _cols(t: torch.Tensor, rank: int, tp: int) -> torch.Tensor:
    n = t.shape[1] // tp
    return t[:, rank * n:(rank + 1) * n]


def load_from_hf_checkpoint(model, path: str, strict=False, parallel_context=None) -> Tuple[int, int]:
    """Copy the weights under ``path`` into ``model`` (any TP rank / PP stage).  Returns
    ``(loaded, missing)`` parameter counts; missing keys are skipped unless ``strict``.  Shapes are checked for every
    tensor before the first one is copied: a checkpoint of another architecture raises ``ValueError`` naming the tensors
    and leaves the model as it was.  The reference passes its
    parallel context in third place (src/distributed/tensor_parallel.py:947-1064); here the shard to read follows
    from the model's own layout, so a context given there (or as ``parallel_context``) is accepted and not needed."""
    if not isinstance(strict, bool):
        strict = False
    sd = _load_all(path)
    tp, rank = model.tp_size, model.tp_rank
    loaded = missing = 0
    copies, bad = [], []        # (parameter, tensor) to copy once every shape has been checked

    def get(name):
        nonlocal missing
        t = sd.get(name)
        if t is None:
            missing += 1
            if strict:
                raise KeyError(f"{name} not found in {path}")
        return t

    def put(param, t, what=""):
        nonlocal loaded
        if t is None:
            return
        if tuple(param.shape) != tuple(t.shape):
            bad.append(f"{what or 'tensor'}: checkpoint {tuple(t.shape)}, model {tuple(param.shape)}")
            return
        copies.append((param, t))
        loaded += 1

    if model.embed_tokens is not None:
        put(model.embed_tokens, get("model.embed_tokens.weight"), "model.embed_tokens.weight")
    for i, layer in enumerate(model.layers):
        g = f"model.layers.{model.layer_start + i}."
        q, k, v = get(g + "self_attn.q_proj.weight"), get(g + "self_attn.k_proj.weight"), get(g + "self_attn.v_proj.weight")
        if q is not None and k is not None and v is not None:
            put(layer.self_attn.qkv_proj.weight, torch.cat([_rows(q, rank, tp), _rows(k, rank, tp), _rows(v, rank, tp)], 0),
                g + "self_attn.{q,k,v}_proj.weight")
            loaded += 2
        o = get(g + "self_attn.o_proj.weight")
        put(layer.self_attn.o_proj.weight, None if o is None else _cols(o, rank, tp), g + "self_attn.o_proj.weight")
        put(layer.self_attn.q_norm.weight, get(g + "self_attn.q_norm.weight"), g + "self_attn.q_norm.weight")
        put(layer.self_attn.k_norm.weight, get(g + "self_attn.k_norm.weight"), g + "self_attn.k_norm.weight")
        gate, up = get(g + "mlp.gate_proj.weight"), get(g + "mlp.up_proj.weight")
        if gate is not None and up is not None:
            put(layer.mlp.gate_up_proj.weight, torch.cat([_rows(gate, rank, tp), _rows(up, rank, tp)], 0),
                g + "mlp.{gate,up}_proj.weight")
            loaded += 1
        down = get(g + "mlp.down_proj.weight")
        put(layer.mlp.down_proj.weight, None if down is None else _cols(down, rank, tp), g + "mlp.down_proj.weight")
        put(layer.input_layernorm.weight, get(g + "input_layernorm.weight"), g + "input_layernorm.weight")
        put(layer.post_attention_layernorm.weight, get(g + "post_attention_layernorm.weight"),
            g + "post_attention_layernorm.weight")
    if model.norm is not None:
        put(model.norm.weight, get("model.norm.weight"), "model.norm.weight")
    if model.lm_head is not None:
        t = sd.get("lm_head.weight")
        if t is None:
            t = sd.get("model.embed_tokens.weight")  # tied checkpoints omit lm_head
        if t is not None and getattr(model, "vocab_parallel", False):
            t = _rows(t, rank, tp)
        put(model.lm_head, t, "lm_head.weight")
    if bad:
        raise ValueError(f"{path} does not fit this model ({len(bad)} tensors), nothing was loaded: " + "; ".join(bad[:4])
                         + (" ..." if len(bad) > 4 else ""))
    with torch.no_grad():
        for param, t in copies:
            param.copy_(t.to(param.dtype))
    return loaded, missing


def hf_named_tensors(model, gather_tp: bool = True, merge_lora: bool = False) -> Iterator[Tuple[str, torch.Tensor]]:
    """Yield ``(hf_name, full_tensor)`` for this stage's weights.  With TP>1 and ``gather_tp`` the
    shards are all-gathered over the TP group so every rank sees full tensors.  ``merge_lora`` yields
    ``W + scaling * B A`` for adapted projections, built out of place (the live base weights stay as they are)."""
    import torch.distributed as dist

    tp, group = model.tp_size, model.tp_group
    cfg = model.cfg
    D = cfg.head_dim

    def gather(t, dim):
        if tp == 1 or not gather_tp:
            return t
        parts = [torch.empty_like(t) for _ in range(tp)]
        dist.all_gather(parts, t.contiguous(), group=group)
        return torch.cat(parts, dim=dim)

    def weight_of(mod):
        if merge_lora and hasattr(mod, "merged_weight"):
            return mod.merged_weight()
        return mod.weight.detach()

    if model.embed_tokens is not None:
        yield "model.embed_tokens.weight", model.embed_tokens.detach()
    for i, layer in enumerate(model.layers):
        g = f"model.layers.{model.layer_start + i}."
        hq, hk = layer.self_attn.heads_local * D, layer.self_attn.kv_heads_local * D
        w = weight_of(layer.self_attn.qkv_proj)
        yield g + "self_attn.q_proj.weight", gather(w[:hq], 0)
        yield g + "self_attn.k_proj.weight", gather(w[hq:hq + hk], 0)
        yield g + "self_attn.v_proj.weight", gather(w[hq + hk:], 0)
        yield g + "self_attn.o_proj.weight", gather(weight_of(layer.self_attn.o_proj), 1)
        yield g + "self_attn.q_norm.weight", layer.self_attn.q_norm.weight.detach()
        yield g + "self_attn.k_norm.weight", layer.self_attn.k_norm.weight.detach()
        gu = weight_of(layer.mlp.gate_up_proj)
        il = gu.shape[0] // 2
        yield g + "mlp.gate_proj.weight", gather(gu[:il], 0)
        yield g + "mlp.up_proj.weight", gather(gu[il:], 0)
        yield g + "mlp.down_proj.weight", gather(weight_of(layer.mlp.down_proj), 1)
        yield g + "input_layernorm.weight", layer.input_layernorm.weight.detach()
        yield g + "post_attention_layernorm.weight", layer.post_attention_layernorm.weight.detach()
    if model.norm is not None:
        yield "model.norm.weight", model.norm.weight.detach()
    if model.is_last_stage and not model.tied:
        w = model.lm_head.detach()
        yield "lm_head.weight", gather(w, 0) if getattr(model, "vocab_parallel", False) else w


def save_hf_checkpoint(model, path: str, write: bool = True, shard_name: str = "model.safetensors") -> None:
    """Write this stage's weights with HF names.  Collective over the TP group when TP>1 (call it on
    every TP rank; pass ``write=False`` on the ranks that should not touch the file system)."""
    from safetensors.torch import save_file

    tensors = {k: v.to("cpu").contiguous().clone() for k, v in hf_named_tensors(model)}
    if write:
        write_hf_config(path, model.cfg)
        save_file(tensors, os.path.join(path, shard_name), metadata={"format": "pt"})
