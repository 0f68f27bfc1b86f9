"""Weight sync by chunked NVLink peer writes.

The trainer casts and writes every (merged) weight straight into a *staging* buffer that lives in the
inference GPU's memory (``b2_peer_write``: cast + optional in-place add + running checksum, one launch
per chunk), then publishes ``{version, checksum}``.  The engine recomputes the checksum over its
staging buffer; only if it matches does it copy staging -> live parameters (a device-local copy, so the
parameter addresses captured in CUDA graphs stay valid) and bump its version; on a mismatch it keeps
the previous weights and reports the failure.  SwiftSync LoRA deltas use the same kernel in add mode
against an fp32 staging image of the adapter state.

Transport: between processes the staging buffer is a symmetric-memory allocation
(``torch.distributed._symmetric_memory``) whose peer pointer the trainer writes through; inside one
process (colocated trainer and engine on one GPU) the "peer" pointer is simply local.  The control
message (layout once, then version + checksum per sync) travels over the process group.
Replaces CUDA-IPC-over-HTTP, per-tensor NCCL broadcast and the Ray object store
(src/transfer/ipc_transfer.py:290-563, src/transfer/nccl_transfer.py:76-361).
"""
from __future__ import annotations

import time
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from .. import _native as nv
from ..obs import nvtx
from ..obs.logging import get_logger
from .nccl_transfer import TransferStats

logger = get_logger("sync.peer_write")

MASK64 = (1 << 64) - 1


def fletcher_checksum(t: torch.Tensor, elem_offset: int = 0) -> Tuple[int, int]:
    """Host oracle of the device checksum: (sum of element bit patterns, sum of pattern * (index+1)),
    both mod 2^64, over a bf16 or fp32 tensor."""
    flat = t.detach().reshape(-1).cpu()
    if flat.dtype == torch.bfloat16:
        bits = flat.view(torch.int16).to(torch.int64) & 0xFFFF
    else:
        bits = flat.to(torch.float32).view(torch.int32).to(torch.int64) & 0xFFFFFFFF
    c0 = int(bits.sum().item()) & MASK64
    c1 = 0
    idx = torch.arange(1 + elem_offset, 1 + elem_offset + bits.numel(), dtype=torch.int64)
    for s in range(0, bits.numel(), 1 << 16):     # python ints: exact modulo 2^64
        c1 = (c1 + sum(int(b) * int(i) for b, i in zip(bits[s:s + (1 << 16)].tolist(),
                                                       idx[s:s + (1 << 16)].tolist()))) & MASK64
    return c0, c1


def device_checksum(t: torch.Tensor) -> Tuple[int, int]:
    if not t.is_cuda:
        return fletcher_checksum(t)
    out = torch.zeros(2, dtype=torch.int64, device=t.device)
    nv.check(nv.lib().b2_words_checksum(nv.ptr(t), int(t.dtype == torch.float32), nv.ctypes.c_longlong(t.numel()),
                                        nv.ptr(out), nv.stream_ptr()), "words_checksum")
    nv.count_launch()
    a, b = out.tolist()
    return a & MASK64, b & MASK64


class VersionedWeightBuffer:
    """Engine-side staging image of a set of named tensors in one flat buffer, plus the version."""

    def __init__(self, layout: List[Tuple[str, Tuple[int, ...]]], dtype: torch.dtype, device,
                 storage: Optional[torch.Tensor] = None):
        self.layout, self.dtype = layout, dtype
        self.offsets: Dict[str, Tuple[int, int, Tuple[int, ...]]] = {}
        n = 0
        for name, shape in layout:
            cnt = 1
            for d in shape:
                cnt *= d
            self.offsets[name] = (n, cnt, tuple(shape))
            n += (cnt + 7) // 8 * 8
        self.numel = max(n, 8)
        self.flat = storage if storage is not None else torch.zeros(self.numel, dtype=dtype, device=device)
        assert self.flat.numel() >= self.numel
        self.version = 0
        self.rejected = 0

    def view(self, name: str) -> torch.Tensor:
        o, cnt, shape = self.offsets[name]
        return self.flat[o:o + cnt].view(shape)

    def named_views(self) -> Dict[str, torch.Tensor]:
        return {k: self.view(k) for k in self.offsets}

    def verify_and_commit(self, version: int, checksum: Tuple[int, int], apply) -> bool:
        """Compare the checksum of the staged bytes; on success call ``apply(named_views)`` (copies into
        the live parameters) and adopt ``version``; otherwise keep the old version."""
        got = device_checksum(self.flat[:self.numel])
        if (got[0], got[1]) != (checksum[0] & MASK64, checksum[1] & MASK64):
            self.rejected += 1
            return False
        apply(self.named_views())
        self.version = version
        return True


class PeerWeightSync:
    """Both ends of the peer-write sync.  A full sync is verified against the checksum of the whole staged image;
    a delta (``add=True``) against the checksum of exactly the spans it touched, which the control message lists.

    ``sender_rank`` writes, ``receiver_ranks`` each own a staging buffer.  With ``group=None`` the sync
    is process-local (trainer and engine share the GPU): ``staging`` is then an ordinary tensor.
    """

    UNIT = 1 << 20        # elements per unit of the batched write

    def __init__(self, layout: List[Tuple[str, Tuple[int, ...]]], dtype: torch.dtype = torch.bfloat16, device=None,
                 group=None, sender_rank: int = 0, chunk_elems: int = 1 << 24):
        self.device = device if device is not None else (
            torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu"))
        self.group, self.sender_rank, self.chunk = group, sender_rank, chunk_elems
        self.rank = dist.get_rank(group) if group is not None else 0
        self.world = dist.get_world_size(group) if group is not None else 1
        self.stats = TransferStats()
        self.version = 0
        self.peer_ptrs: Optional[List[int]] = None
        storage = None
        probe = VersionedWeightBuffer(layout, dtype, "meta")
        if group is not None and self.device.type == "cuda":
            import torch.distributed._symmetric_memory as symm
            storage = symm.empty(probe.numel, dtype=dtype, device=self.device)
            hdl = symm.rendezvous(storage, group=group)
            self.peer_ptrs = [int(p) for p in hdl.buffer_ptrs]
            self._hdl = hdl
            storage.zero_()
        self.staging = VersionedWeightBuffer(layout, dtype, self.device, storage)
        self._cks = torch.zeros(2, dtype=torch.int64, device=self.device) if self.device.type == "cuda" else None
        self.last_spans: List[Tuple[int, int]] = []

    # ---- sender ------------------------------------------------------------------------------------------
    def _dst_ptr(self, target_rank: Optional[int]) -> int:
        if self.peer_ptrs is None or target_rank is None:
            return self.staging.flat.data_ptr()
        return self.peer_ptrs[target_rank]

    def write(self, state: Dict[str, torch.Tensor], target_rank: Optional[int] = None, add: bool = False
              ) -> Tuple[Tuple[int, int], int]:
        """Write ``state`` into the target's staging buffer.  Returns ((c0, c1), bytes)."""
        st = self.staging
        nbytes = 0
        if self.device.type != "cuda":
            self.last_spans = []
            for k, v in state.items():
                if k not in st.offsets:
                    raise KeyError(f"peer write: {k!r} is not part of the staging layout")
                if v.numel() < st.offsets[k][1]:
                    raise ValueError(f"peer write: {k!r} has {v.numel()} elements, the staging layout holds {st.offsets[k][1]}")
                dst = st.view(k)
                v = v.reshape(-1)[:dst.numel()].reshape(dst.shape)
                dst.copy_((dst.float() + v.float()).to(st.dtype) if add else v.to(st.dtype))
                nbytes += v.numel() * st.flat.element_size()
                self.last_spans.append(st.offsets[k][:2])
            return (self.spans_checksum(self.last_spans) if add else fletcher_checksum(st.flat[:st.numel])), nbytes
        self._cks.zero_()
        base = self._dst_ptr(target_rank)
        es = st.flat.element_size()
        L = nv.lib()
        # one launch for the whole image (two when the sources mix fp32 and bf16): a table of
        # (source pointer, destination offset, element count) units, large tensors cut into UNIT-element pieces
        keep, by_dtype = [], {True: [], False: []}
        for k, v in state.items():
            if k not in st.offsets:
                raise KeyError(f"peer write: {k!r} is not part of the staging layout")
            off, cnt, _ = st.offsets[k]
            if v.numel() < cnt:
                # the kernel reads `cnt` elements from the source pointer: a shorter tensor would be read past its end
                raise ValueError(f"peer write: {k!r} has {v.numel()} elements, the staging layout holds {cnt}")
            if v.numel() > cnt:
                logger.warning("peer write: %r has %d elements, only the first %d fit the staging layout", k, v.numel(), cnt)
            if v.device.type != self.device.type or (v.device.index is not None and self.device.index is not None
                                                     and v.device.index != self.device.index):
                raise ValueError(f"peer write: {k!r} lives on {v.device}, the writer runs on {self.device}")
            src = v.detach().reshape(-1)
            if src.dtype not in (torch.float32, torch.bfloat16):
                src = src.float()
            src = src.contiguous()
            keep.append(src)                       # alive until the host sync below
            sz, ptr0 = src.element_size(), src.data_ptr()
            rows = by_dtype[src.dtype == torch.float32]
            for s0 in range(0, cnt, self.UNIT):
                rows.append((ptr0 + s0 * sz, off + s0, min(self.UNIT, cnt - s0)))
            nbytes += cnt * es
        self.last_spans = [(off, n) for rows in by_dtype.values() for _, off, n in rows]
        for is_fp32, rows in by_dtype.items():
            if not rows:
                continue
            table = torch.tensor(rows, dtype=torch.int64).pin_memory().to(self.device, non_blocking=True)
            keep.append(table)
            nv.check(L.b2_peer_write_batch(nv.ptr(table), len(rows), int(is_fp32), nv.ctypes.c_void_p(base),
                                           int(st.dtype == torch.float32), int(add), nv.ptr(self._cks),
                                           nv.stream_ptr()), "peer_write_batch")
            nv.count_launch()
        # padding between tensors is zero on both sides and contributes nothing to either sum
        a, b = self._cks.tolist()      # synchronises: every write has been issued and fenced
        return (a & MASK64, b & MASK64), nbytes

    def spans_checksum(self, spans) -> Tuple[int, int]:
        """Checksum of the given ``(element offset, count)`` spans of this rank's staging image (what a delta
        touched), with the same position weights the writer used."""
        st = self.staging
        if self.device.type != "cuda":
            c0 = c1 = 0
            for off, n in spans:
                a, b = fletcher_checksum(st.flat[off:off + n], off)
                c0, c1 = (c0 + a) & MASK64, (c1 + b) & MASK64
            return c0, c1
        out = torch.zeros(2, dtype=torch.int64, device=self.device)
        table = torch.tensor([(0, off, n) for off, n in spans], dtype=torch.int64).pin_memory().to(self.device, non_blocking=True)
        nv.check(nv.lib().b2_spans_checksum(nv.ptr(table), len(spans), nv.ptr(st.flat),
                                            int(st.dtype == torch.float32), nv.ptr(out), nv.stream_ptr()),
                 "spans_checksum")
        nv.count_launch()
        a, b = out.tolist()
        return a & MASK64, b & MASK64

    # ---- protocol ------------------------------------------------------------------------------------------
    @nvtx.annotate("sync/peer_write")
    def sync(self, is_sender: bool, state: Optional[Dict[str, torch.Tensor]] = None, engine=None,
             add: bool = False, corrupt: bool = False) -> int:
        """One full sync.  Process-local when there is no group.  ``corrupt`` flips the announced
        checksum (host-side fault injection for the rejection path)."""
        t0 = time.perf_counter()
        apply = (lambda views: engine.load_weights(views)) if engine is not None else (lambda views: None)
        if self.group is None:
            cks, nbytes = self.write(state, None, add)
            if corrupt:
                cks = (cks[0] ^ 1, cks[1])
            if add:           # a delta's checksum covers exactly the spans it touched
                ok = self.spans_checksum(self.last_spans) == (cks[0] & MASK64, cks[1] & MASK64)
                if ok:
                    apply(self.staging.named_views())
                    self.staging.version = self.version + 1
                else:
                    self.staging.rejected += 1
            else:
                ok = self.staging.verify_and_commit(self.version + 1, cks, apply)
            self.stats.record(nbytes, time.perf_counter() - t0, ok)
            if ok:
                self.version += 1
            return self.version
        if is_sender:
            msgs = {}
            nbytes = 0
            for r in range(self.world):
                if r == self.rank:
                    continue
                cks, nb = self.write(state, r, add)
                msgs[r] = cks if not corrupt else (cks[0] ^ 1, cks[1])
                nbytes += nb
            box = [{"version": self.version + 1, "checksums": msgs, "add": add, "spans": self.last_spans if add else None}]
            dist.broadcast_object_list(box, src=dist.get_global_rank(self.group, self.sender_rank), group=self.group)
            acks = [None] * self.world
            dist.all_gather_object(acks, True, group=self.group)
            ok = all(a for a in acks)
            self.stats.record(nbytes, time.perf_counter() - t0, ok)
            if ok:
                self.version += 1
            return self.version
        box = [None]
        dist.broadcast_object_list(box, src=dist.get_global_rank(self.group, self.sender_rank), group=self.group)
        msg = box[0]
        cks = msg["checksums"][self.rank]
        if msg["add"]:
            # the writer's checksum is over the values it stored into exactly these spans: a corrupted delta is
            # rejected like a corrupted full image (the additions have landed in staging, the live weights and the
            # version stay as they were; the next full sync rewrites staging)
            ok = self.spans_checksum(msg["spans"]) == (cks[0] & MASK64, cks[1] & MASK64)
            if ok:
                apply(self.staging.named_views())
                self.staging.version = msg["version"]
            else:
                self.staging.rejected += 1
        else:
            ok = self.staging.verify_and_commit(msg["version"], cks, apply)
        acks = [None] * self.world
        dist.all_gather_object(acks, ok, group=self.group)
        if ok and all(a for a in acks):
            self.version = msg["version"]
        self.stats.record(0, time.perf_counter() - t0, ok)
        return self.version

    def get_stats(self) -> Dict:
        return {"version": self.version, "transfers": self.stats.transfers, "failures": self.stats.failures,
                "rejected": self.staging.rejected, "avg_gbps": self.stats.avg_gbps, "last_gbps": self.stats.last_gbps}
