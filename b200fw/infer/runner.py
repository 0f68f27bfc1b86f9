"""ModelRunner: runs the framework's own Qwen3 weights over the paged KV cache.

Where the reference wraps a Hugging Face model and moves KV between its ``DynamicCache`` and the pages
with Python loops (src/inference/model_runner.py:192-433), this runner drives the native layers
directly: fused QKV GEMM -> QK-norm + RoPE kernel -> KV-store kernel -> paged decode / variable-length
prefill attention -> GEMMs with the residual in the epilogue.  It also builds the per-step metadata
(store segments, block tables, cu_seqlens, gather slots) in pinned host memory.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import torch

from .. import ops
from ..model.qwen3 import ParallelTransformerModel
from .context import InferenceContext
from .kv_cache import BlockPool, KVCacheManager


@dataclass
class ModelRunnerConfig:
    """Model-side slice of ``InferenceConfig`` (src/inference/model_runner.py:32-47); ``from_runner`` fills it
    from a live runner."""
    num_layers: int = 32
    num_heads: int = 32
    num_kv_heads: int = 8
    head_dim: int = 128
    hidden_size: int = 4096
    vocab_size: int = 151936
    block_size: int = 16
    max_num_blocks: int = 1024
    dtype: torch.dtype = torch.bfloat16
    device: str = "cuda"
    enable_cuda_graph: bool = True
    max_cuda_graph_batch_size: int = 64

    @classmethod
    def from_runner(cls, r: "ModelRunner") -> "ModelRunnerConfig":
        c = r.cfg
        return cls(c.num_layers, c.num_heads, c.num_kv_heads, c.head_dim, c.hidden_size, c.vocab_size, r.block_size,
                   r.pool.num_blocks, r.dtype, str(r.device), getattr(r, "graph_runner", None) is not None)


class ModelRunner:
    def __init__(self, model: ParallelTransformerModel, pool: BlockPool, manager: KVCacheManager,
                 partition_size: int = 512, enable_partitioned: bool = False):
        assert model.tp_size == 1, "the inference runner drives one GPU per engine instance"
        self.model, self.pool, self.mgr = model, pool, manager
        self.cfg = model.cfg
        self.device = next(model.parameters()).device
        self.dtype = next(model.parameters()).dtype
        self.partition_size, self.enable_partitioned = partition_size, enable_partitioned
        self.block_size = pool.block_size
        self.forward_calls = 0
        self.fuse_kv_store = True     # norm + RoPE + cache store in one launch for 16-bit caches (False: two launches)

    # ---- metadata ----------------------------------------------------------------------------------------
    def _stage(self, t: torch.Tensor) -> torch.Tensor:
        """Host tensor -> device through a ring of reusable pinned buffers.  Page-locking a fresh buffer per tensor
        costs more than the copy; a ring (not one buffer) because the engine queues a step's copies while the GPU
        may still be running the previous step, whose staging memory must stay untouched until its copy has run."""
        if self.device.type != "cuda":
            return t
        n = t.numel() * t.element_size()
        ring = self.__dict__.setdefault("_rings", {})
        r = ring.setdefault(t.dtype, {"bufs": [None] * 16, "i": 0})
        i = r["i"] = (r["i"] + 1) % len(r["bufs"])
        if r["bufs"][i] is None or r["bufs"][i].numel() < t.numel():
            r["bufs"][i] = torch.empty(max(1024, t.numel()), dtype=t.dtype, pin_memory=True)
        view = r["bufs"][i][:t.numel()].view(t.shape)
        view.copy_(t)
        return view.to(self.device, non_blocking=True)

    def _dev(self, data, dtype) -> torch.Tensor:
        return self._stage(torch.tensor(data, dtype=dtype))

    @staticmethod
    def _segments(table: List[int], start: int, count: int, row0: int, bs: int) -> List[List[int]]:
        """Split positions [start, start+count) of one sequence into per-block runs."""
        segs, pos, row = [], start, row0
        end = start + count
        while pos < end:
            off = pos % bs
            n = min(bs - off, end - pos)
            segs.append([table[pos // bs], row, n, off])
            pos += n
            row += n
        return segs

    def prepare_prefill(self, seq_ids: Sequence, starts: Sequence[int], counts: Sequence[int]) -> InferenceContext:
        """Metadata for a batch of prefill chunks: sequence ``i`` computes positions
        ``starts[i] .. starts[i]+counts[i]`` (its KV blocks must already cover them)."""
        bs = self.block_size
        cu_q, cu_k, segs, pos, slots, last = [0], [0], [], [], [], []
        need_gather = any(s > 0 for s in starts)
        # a bf16 cache is read in place through the block table; only an fp8 cache (dequantised) is gathered
        paged = need_gather and self.device.type == "cuda" and not self.pool.fp8
        tables = []
        new_slots = []                                   # cache row of every new token (the fused norm + RoPE + store)
        for sid, st, n in zip(seq_ids, starts, counts):
            table = self.mgr.get_block_table(sid)
            segs += self._segments(table, st, n, cu_q[-1], bs)
            pos += list(range(st, st + n))
            new_slots += [table[p // bs] * bs + p % bs for p in range(st, st + n)]
            if paged:
                tables.append(table[:(st + n + bs - 1) // bs])
            elif need_gather:
                slots += [table[p // bs] * bs + p % bs for p in range(st + n)]
            cu_q.append(cu_q[-1] + n)
            cu_k.append(cu_k[-1] + (st + n if need_gather else n))
            last.append(cu_q[-1] - 1)
        bt = None
        if paged:
            width = max(len(t) for t in tables)
            bt = self._dev([list(t) + [0] * (width - len(t)) for t in tables], torch.int32)
        return InferenceContext(
            is_prefill=True, num_seqs=len(seq_ids), store_segments=self._dev(segs, torch.int32),
            cu_seqlens_q=self._dev(cu_q, torch.int32), cu_seqlens_k=self._dev(cu_k, torch.int32),
            max_seqlen_q=max(counts), total_q=cu_q[-1], total_k=cu_k[-1],
            gather_slots=self._dev(slots, torch.int32) if (need_gather and not paged) else None,
            block_tables=bt, positions=self._dev(pos, torch.int32), last_token_rows=self._dev(last, torch.long),
            slot_mapping=self._dev(new_slots, torch.int32))

    def prepare_decode(self, seq_ids: Sequence, pad_to: int = 0, max_blocks: int = 0) -> InferenceContext:
        """Metadata for one decode step: every sequence's newest token sits at position ``len-1`` (its
        slot must already be allocated with ``append_token``)."""
        import numpy as np
        bs = self.block_size
        n = len(seq_ids)
        B = max(n, pad_to)
        tables = [self.mgr.tables[s] for s in seq_ids]
        lens = np.fromiter((t.num_tokens for t in tables), dtype=np.int32, count=n)
        width = max(max_blocks, max((t.num_blocks for t in tables), default=1), 1)
        bt = np.full((B, width), -1, dtype=np.int32)
        for i, t in enumerate(tables):
            ids = t.get_physical_block_ids()
            bt[i, :len(ids)] = ids
        segs = np.zeros((B, 4), dtype=np.int32)
        segs[:, 0] = -1
        if n:
            last = lens - 1
            segs[:n, 0] = bt[np.arange(n), last // bs]
            segs[:n, 1] = np.arange(n)
            segs[:n, 2] = 1
            segs[:n, 3] = last % bs
        slots = np.full(B, -1, dtype=np.int32)
        if n:
            slots[:n] = segs[:n, 0] * bs + segs[:n, 3]
        ctx_lens = np.zeros(B, dtype=np.int32)
        ctx_lens[:n] = lens
        pos = np.zeros(B, dtype=np.int32)
        pos[:n] = lens - 1

        def dev(a):
            return self._stage(torch.from_numpy(a))

        return InferenceContext(
            is_prefill=False, num_seqs=B, block_tables=dev(bt), context_lens=dev(ctx_lens),
            max_context_len=int(lens.max()) if n else 0, store_segments=dev(segs), positions=dev(pos),
            slot_mapping=dev(slots))

    # ---- forward -----------------------------------------------------------------------------------------
    def _split_plan(self, ctx: InferenceContext) -> Tuple[int, int]:
        if self.enable_partitioned and ctx.max_context_len > self.partition_size:
            part = max(64, self.partition_size // 64 * 64)
            return part, (ctx.max_context_len + part - 1) // part
        if getattr(self, "balance_splits", False) and ctx.max_context_len > 256:
            # One CTA per (sequence, kv head group) leaves the last of ~3.5 waves (256 sequences x 8 kv heads over
            # 148 SMs x 4 resident CTAs) mostly empty, and a long sequence pins its CTA while the others finish.
            # Splitting every sequence into a few partitions gives ~8 waves of shorter CTAs; the exact log-sum-exp
            # merge costs one small kernel.
            cfg = self.cfg
            g = cfg.num_heads // cfg.num_kv_heads
            gh = 4 if g % 4 == 0 and not self.pool.fp8 else (2 if g % 2 == 0 else 1)
            ctas = ctx.num_seqs * cfg.num_kv_heads * (g // gh)
            want = 8 * 148 * 4
            if ctas < want:
                nsplit = min((ctx.max_context_len + 255) // 256, -(-want // ctas))
                if nsplit > 1:
                    part = -(-ctx.max_context_len // nsplit)
                    part = (part + 63) // 64 * 64
                    return part, (ctx.max_context_len + part - 1) // part
        return 0, 1

    @torch.no_grad()
    def forward(self, token_ids: torch.Tensor, ctx: InferenceContext, all_rows: bool = False,
                split_plan: Optional[Tuple[int, int]] = None) -> torch.Tensor:
        """Token ids ``[T]`` -> logits ``[num_seqs, V]`` of each sequence's last row (or of every row)."""
        m, cfg = self.model, self.cfg
        self.forward_calls += 1
        Hq, Hkv, D = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim
        cos, sin = ops.rope_tables(cfg.max_position_embeddings, D, cfg.rope_theta, self.device)
        part, nsplit = split_plan if split_plan is not None else (self._split_plan(ctx) if not ctx.is_prefill else (0, 1))
        h = ops.embedding(token_ids, m.embed_tokens)
        # a 16-bit cache takes the new rows straight from the norm + RoPE kernel; the fp8 cache keeps its own store
        # kernel (it maintains the per-block scale and requantises a block when the scale grows)
        fused_store = (self.fuse_kv_store and not self.pool.fp8 and ctx.slot_mapping is not None
                       and ctx.slot_mapping.dtype == torch.int32 and (D == 128 or self.device.type != "cuda"))
        for li, layer in enumerate(m.layers):
            att_mod = layer.self_attn
            x = ops.rmsnorm(h, layer.input_layernorm.weight, cfg.rms_norm_eps)
            qkv = ops.linear(x, att_mod.qkv_proj.weight)
            kc, vc = self.pool.layer_kv(li)
            ks, vs = self.pool.layer_scales(li)
            if fused_store:
                # split + per-head norm + rotation + store of the new K / V rows: one launch
                q, k, v = ops.qknorm_rope_store(qkv, att_mod.q_norm.weight, att_mod.k_norm.weight, ctx.positions, cos, sin,
                                                Hq, Hkv, D, cfg.rms_norm_eps, kc, vc, ctx.slot_mapping)
            else:
                q, k, v = ops.qknorm_rope(qkv, att_mod.q_norm.weight, att_mod.k_norm.weight, ctx.positions, cos, sin,
                                          Hq, Hkv, D, cfg.rms_norm_eps)
                ops.kv_store(k, v, kc, vc, ctx.store_segments, ks, vs)
            if ctx.is_prefill:
                if ctx.block_tables is not None:
                    # chunks with earlier context: keys / values are read in place through the block table
                    att = ops.paged_prefill_attention(q, kc, vc, ctx.block_tables, ctx.cu_seqlens_q, ctx.cu_seqlens_k,
                                                      ctx.max_seqlen_q, Hq)
                else:
                    if ctx.gather_slots is not None:
                        K, V = ops.kv_gather(kc, vc, ctx.gather_slots, self.dtype, ks, vs)
                    else:
                        K, V = k, v
                    att = ops.varlen_attention(q, K, V, ctx.cu_seqlens_q, ctx.cu_seqlens_k, ctx.max_seqlen_q, Hq, Hkv)
            else:
                att = ops.paged_decode_attention(q, kc, vc, ctx.block_tables, ctx.context_lens, Hq,
                                                 k_scale=ks, v_scale=vs, partition=part, nsplit=nsplit)
            h = ops.linear(att, att_mod.o_proj.weight, h)
            x = ops.rmsnorm(h, layer.post_attention_layernorm.weight, cfg.rms_norm_eps)
            gu = ops.linear(x, layer.mlp.gate_up_proj.weight)
            h = ops.linear(ops.swiglu(gu), layer.mlp.down_proj.weight, h)
        if ctx.is_prefill and not all_rows:
            h = h.index_select(0, ctx.last_token_rows)
        h = ops.rmsnorm(h.contiguous(), m.norm.weight, cfg.rms_norm_eps)
        return m.logits_from_hidden(h)

    # ---- the reference's entry points (src/inference/model_runner.py:82-160, 639-812) ----------------------------
    def run(self, input_ids: torch.Tensor, ctx_or_positions=None, is_prefill: bool = True) -> torch.Tensor:
        """``run(token_ids, ctx)``; or, in the reference's style, ``run(token_ids, positions, is_prefill)`` after
        ``b200fw.infer.context.set_context(...)`` published the step's metadata."""
        if isinstance(ctx_or_positions, InferenceContext):
            return self.forward(input_ids.reshape(-1), ctx_or_positions)
        from .context import get_context
        ctx = get_context()
        if ctx is None:
            raise RuntimeError("no InferenceContext: pass one, or call set_context() first")
        if ctx.positions is None and ctx_or_positions is not None:
            ctx.positions = ctx_or_positions.to(torch.int32)
        return self.forward(input_ids.reshape(-1), ctx)

    def run_batch_decode(self, input_ids: torch.Tensor, positions: torch.Tensor, block_tables: torch.Tensor,
                         context_lens: torch.Tensor) -> torch.Tensor:
        """One decode token for every sequence from raw metadata tensors: ``input_ids [B]`` or ``[B,1]``,
        ``positions [B]`` (index of the new token), ``block_tables [B, max_blocks]`` (``-1`` padded),
        ``context_lens [B]`` (including the new token).  Returns ``[B, V]`` logits; the new K/V rows are written
        to ``block_tables[b, positions[b] // block_size]``."""
        B = input_ids.shape[0]
        dev, bs = self.device, self.block_size
        pos = positions.to(dev, torch.int64)
        bt = block_tables.to(dev, torch.int32)
        blk = bt.gather(1, (pos // bs)[:, None]).squeeze(1)
        rows = torch.arange(B, device=dev, dtype=torch.int32)
        seg = torch.stack([blk, rows, torch.ones_like(rows), (pos % bs).to(torch.int32)], 1).contiguous()
        slots = (blk.to(torch.int64) * bs + pos % bs).to(torch.int32)
        lens = context_lens.to(dev, torch.int32)
        ctx = InferenceContext(is_prefill=False, num_seqs=B, block_tables=bt.contiguous(), context_lens=lens,
                               max_context_len=int(lens.max()) if B else 0, store_segments=seg,
                               positions=pos.to(torch.int32), slot_mapping=slots)
        return self.forward(input_ids.reshape(-1).to(dev), ctx)

    def bind_kv_cache(self, pool: BlockPool, manager: Optional[KVCacheManager] = None):
        """Point the runner at another block pool (and its manager)."""
        self.pool, self.block_size = pool, pool.block_size
        if manager is not None:
            self.mgr = manager

    def bind_hf_model(self, model):
        """Swap the model the runner drives.  It has to be this framework's ``ParallelTransformerModel`` (load a
        Hugging Face checkpoint into one with ``load_from_hf_checkpoint``): the kernels address its fused
        projection weights directly, a ``transformers`` module cannot be driven."""
        if not isinstance(model, ParallelTransformerModel):
            raise TypeError("ModelRunner drives a ParallelTransformerModel; load the HF checkpoint into one with "
                            "b200fw.model.load_from_hf_checkpoint")
        self.model, self.cfg = model, model.cfg
        self.device, self.dtype = next(model.parameters()).device, next(model.parameters()).dtype

    def capture_cuda_graphs(self, batch_sizes: Optional[List[int]] = None) -> List[int]:
        """Decode graphs are captured lazily, per batch-size bucket, by the engine's ``CUDAGraphRunner`` the first
        time a bucket is used; this returns the buckets that would be used for ``batch_sizes``."""
        gr = getattr(self, "graph_runner", None)
        if gr is None:
            return []
        sizes = batch_sizes or gr.sizes
        return sorted({gr.padded_size(b) for b in sizes if gr.padded_size(b) is not None})

    def invalidate_cuda_graphs(self):
        gr = getattr(self, "graph_runner", None)
        if gr is not None:
            gr.invalidate()

    # ---- sampling ------------------------------------------------------------------------------------------
    def sample(self, logits: torch.Tensor, temperature: torch.Tensor, top_p: torch.Tensor,
               generator: Optional[torch.Generator] = None, return_logprob: bool = False):
        u = torch.rand(logits.shape[0], device=logits.device, generator=generator)
        return ops.topp_sample(logits, temperature, top_p, u, return_logprob)
