"""Collective weight transfer baselines and the backend-agnostic manager.

``NCCLWeightTransfer`` is the measured baseline for sync latency: names are agreed once, every tensor
is broadcast from the trainer rank into template buffers, a checksum over a sample of each tensor is
compared and a version number follows (src/transfer/nccl_transfer.py:76-223).  It runs over whatever
backend the process group has (NCCL on GPUs, gloo in the CPU tests).  ``RayObjectStoreTransfer`` keeps
the reference's interface; Ray is not part of this framework's runtime, so it reports unavailable
unless ``ray`` can be imported.  ``WeightTransferManager`` selects a backend and keeps stats.
"""
from __future__ import annotations

import hashlib
import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch
import torch.distributed as dist
from ..compat import kwarg_aliases


@dataclass
class TransferStats:
    transfers: int = 0
    total_bytes: int = 0
    total_time_s: float = 0.0
    failures: int = 0
    last_gbps: float = 0.0
    history: List[Dict] = field(default_factory=list)

    def record(self, nbytes: int, dt: float, ok: bool = True):
        self.transfers += 1
        self.total_bytes += nbytes
        self.total_time_s += dt
        self.failures += 0 if ok else 1
        self.last_gbps = nbytes / dt / 1e9 if dt > 0 else 0.0
        self.history.append({"bytes": nbytes, "time_s": dt, "gbps": self.last_gbps, "ok": ok})

    @property
    def avg_gbps(self) -> float:
        return self.total_bytes / self.total_time_s / 1e9 if self.total_time_s > 0 else 0.0

    # ---- the reference's field names; its two transfer modules each have a TransferStats with these
    # (src/transfer/ipc_transfer.py:77-102, src/transfer/nccl_transfer.py:57-73) ------------------------------
    total_params: int = 0
    chunks_sent: int = 0
    build_handle_time: float = 0.0
    serialization_time: float = 0.0
    _start_time: float = field(default=0.0, repr=False)

    def start(self):
        self._start_time = time.perf_counter()

    def finish(self):
        """Close the interval opened by ``start`` into ``total_time``."""
        if self._start_time:
            self.total_time_s += time.perf_counter() - self._start_time
            self._start_time = 0.0

    # settable, as the reference's dataclass fields are; when unset they read the measured total
    transfer_time: float = 0.0
    broadcast_time: float = 0.0

    @property
    def total_time(self) -> float:
        return self.total_time_s

    @total_time.setter
    def total_time(self, v: float):
        self.total_time_s = float(v)

    @property
    def sync_count(self) -> int:
        return self.transfers

    @property
    def errors(self) -> int:
        return self.failures

    @property
    def bandwidth_gbps(self) -> float:
        """Bytes over the transfer (or broadcast) time when one was set, else over the total time."""
        t = self.transfer_time or self.broadcast_time or self.total_time_s
        return self.total_bytes / t / 1e9 if t > 0 else 0.0


@dataclass
class WeightVersion:
    """Version stamp of a published weight set (src/transfer/nccl_transfer.py:40-54)."""
    version: int = 0
    timestamp: float = field(default_factory=time.time)
    checksum: str = ""

    def increment(self, checksum: str = "") -> "WeightVersion":
        return WeightVersion(self.version + 1, time.time(), checksum)


def sample_checksum(t: torch.Tensor, n: int = 64) -> str:
    """md5 of the first ``n`` elements (cheap integrity probe, as the reference does)."""
    flat = t.detach().reshape(-1)[:n].to(torch.float32).cpu().contiguous()
    return hashlib.md5(flat.numpy().tobytes()).hexdigest()


class _VersionedMixin:
    """``current_version`` / ``has_new_version`` as in the reference's transfer classes
    (src/transfer/nccl_transfer.py:204-211, 332-351, 480-486): the integer ``version`` wrapped in a
    :class:`WeightVersion` record."""

    @property
    def current_version(self) -> WeightVersion:
        return WeightVersion(int(self.version), self.__dict__.get("_version_time", 0.0), self.__dict__.get("_version_checksum", ""))

    def has_new_version(self, version: int) -> bool:
        return int(self.version) > int(version)

    def get_version_info(self) -> WeightVersion:
        return self.current_version


class NCCLWeightTransfer(_VersionedMixin):
    def __init__(self, group=None, src_rank: int = 0, process_group=None):
        # the reference's order is (src_rank, process_group) (src/transfer/nccl_transfer.py:68-94): an int in first
        # place is the source rank
        if isinstance(group, int) and not isinstance(group, bool):
            group, src_rank = (src_rank if not isinstance(src_rank, int) else None), group
        group = group if group is not None else process_group
        self.group, self.src = group, src_rank
        self.version = 0
        self.stats = TransferStats()
        self._names: Optional[List[str]] = None

    def _bcast_obj(self, obj):
        box = [obj]
        dist.broadcast_object_list(box, src=self.src, group=self.group)
        return box[0]

    @kwarg_aliases(state_dict="state")
    def broadcast_weights(self, state: Dict[str, torch.Tensor]) -> int:
        """Trainer side.  Returns the new version."""
        t0 = time.perf_counter()
        names = list(state.keys())
        meta = self._bcast_obj({"names": names, "shapes": [tuple(state[n].shape) for n in names],
                                "checks": [sample_checksum(state[n]) for n in names]})
        nbytes = 0
        for n in meta["names"]:
            t = state[n].contiguous()
            dist.broadcast(t, src=self.src, group=self.group)
            nbytes += t.numel() * t.element_size()
        self.version = self._bcast_obj(self.version + 1)
        self.stats.record(nbytes, time.perf_counter() - t0)
        return self.version

    def receive_weights(self, templates: Optional[Dict[str, torch.Tensor]] = None, *,
                        state_dict_template: Optional[Dict[str, torch.Tensor]] = None) -> Dict[str, torch.Tensor]:
        """Engine side: receive into ``templates`` (same names / shapes / dtypes; ``state_dict_template`` is the
        reference's keyword for it); verifies the sample checksums and raises on mismatch, leaving ``version``
        unchanged."""
        templates = templates if templates is not None else state_dict_template
        assert templates is not None, "receive_weights needs the template tensors"
        t0 = time.perf_counter()
        meta = self._bcast_obj(None)
        nbytes, bad = 0, []
        for n, shape, chk in zip(meta["names"], meta["shapes"], meta["checks"]):
            buf = templates.get(n)
            if buf is None or tuple(buf.shape) != tuple(shape):
                buf = torch.empty(shape, dtype=next(iter(templates.values())).dtype,
                                  device=next(iter(templates.values())).device)
                templates[n] = buf
            dist.broadcast(buf, src=self.src, group=self.group)
            nbytes += buf.numel() * buf.element_size()
            if sample_checksum(buf) != chk:
                bad.append(n)
        version = self._bcast_obj(None)
        self.stats.record(nbytes, time.perf_counter() - t0, ok=not bad)
        if bad:
            raise RuntimeError(f"weight checksum mismatch for {bad[:3]} ({len(bad)} tensors)")
        self.version = version
        return templates


class RayObjectStoreTransfer(_VersionedMixin):
    """CPU copy -> ``ray.put`` / ``ray.get`` (src/transfer/nccl_transfer.py:226-361)."""

    def __init__(self):
        try:
            import ray  # noqa: F401
            self.available = True
        except ImportError:
            self.available = False
        self.stats = TransferStats()
        self._ref = None
        self.version = 0

    def publish_weights(self, state: Optional[Dict[str, torch.Tensor]] = None, *,
                        state_dict: Optional[Dict[str, torch.Tensor]] = None):
        state = state if state is not None else state_dict          # ``state_dict``: the reference's keyword
        if not self.available:
            raise RuntimeError("ray is not installed: the object-store backend is unavailable")
        import ray
        t0 = time.perf_counter()
        cpu = {k: v.detach().cpu() for k, v in state.items()}
        self._ref = ray.put(cpu)
        self.version += 1
        self.stats.record(sum(v.numel() * v.element_size() for v in cpu.values()), time.perf_counter() - t0)
        return self._ref

    def fetch_weights(self, ref=None, device: str = "cpu") -> Dict[str, torch.Tensor]:
        if not self.available:
            raise RuntimeError("ray is not installed: the object-store backend is unavailable")
        import ray
        state = ray.get(ref if ref is not None else self._ref)
        return {k: v.to(device) for k, v in state.items()}


class WeightTransferManager(_VersionedMixin):
    """One entry point over the backends: ``local`` (same process: in-place copy into the engine),
    ``peer_write`` (NVLink kernel), ``nccl`` (broadcast baseline), ``ray_object_store``."""

    def __init__(self, backend: str = "local", group=None, src_rank: int = 0, peer_sync=None):
        assert backend in ("local", "peer_write", "nccl", "ray_object_store")
        self.backend = backend
        self.nccl = NCCLWeightTransfer(group, src_rank) if backend == "nccl" else None
        self.ray = RayObjectStoreTransfer() if backend == "ray_object_store" else None
        self.peer = peer_sync
        self.stats = TransferStats()
        self.version = 0

    def sync_weights(self, *args, is_sender: Optional[bool] = None, state: Optional[Dict[str, torch.Tensor]] = None,
                     engine=None, templates: Optional[Dict[str, torch.Tensor]] = None,
                     state_dict: Optional[Dict[str, torch.Tensor]] = None,
                     state_dict_template: Optional[Dict[str, torch.Tensor]] = None):
        """``sync_weights(is_sender, state, engine, templates)``; or the reference's call
        ``sync_weights(state_dict, is_sender, state_dict_template)`` (src/transfer/nccl_transfer.py:395-446), told apart
        by what comes first (a flag or a dict of tensors).  Every argument may also be given by keyword under either
        set of names."""
        if args and isinstance(args[0], dict):                      # the reference's order
            names = ("state", "is_sender", "templates")
        else:
            names = ("is_sender", "state", "engine", "templates")
        given = dict(is_sender=is_sender, state=state, engine=engine, templates=templates)
        for name, value in zip(names, args):
            if given[name] is not None:
                raise TypeError(f"sync_weights() got multiple values for argument {name!r}")
            given[name] = value
        is_sender, state, engine, templates = (given[k] for k in ("is_sender", "state", "engine", "templates"))
        is_sender = True if is_sender is None else bool(is_sender)
        state = state if state is not None else state_dict
        templates = templates if templates is not None else state_dict_template
        t0 = time.perf_counter()
        nbytes = sum(v.numel() * v.element_size() for v in state.values()) if state else 0
        if self.backend == "local":
            assert engine is not None and state is not None
            engine.load_weights(state)
            self.version += 1
        elif self.backend == "nccl":
            if is_sender:
                self.version = self.nccl.broadcast_weights(state)
            else:
                out = self.nccl.receive_weights(templates)
                self.version = self.nccl.version
                if engine is not None:
                    engine.load_weights(out)
        elif self.backend == "peer_write":
            self.version = self.peer.sync(is_sender, state, engine)
        else:
            if is_sender:
                self.ray.publish_weights(state)
            elif engine is not None:
                engine.load_weights(self.ray.fetch_weights())
            self.version += 1
        self.stats.record(nbytes, time.perf_counter() - t0)
        return self.version

    async def sync_weights_async(self, *a, **kw):
        import asyncio
        return await asyncio.get_running_loop().run_in_executor(None, lambda: self.sync_weights(*a, **kw))

    def sync_weights_sync(self, state_dict: Optional[Dict[str, torch.Tensor]] = None, is_sender: bool = True,
                          state_dict_template: Optional[Dict[str, torch.Tensor]] = None, engine=None) -> WeightVersion:
        """The reference's blocking entry point and argument order (src/transfer/nccl_transfer.py:448-478): the
        receiver's tensors arrive in ``state_dict_template`` (or ``state_dict``) and are copied into
        ``state_dict`` in place."""
        template = state_dict_template if state_dict_template is not None else state_dict
        self.sync_weights(is_sender, state_dict, engine, templates=None if is_sender else template)
        if not is_sender and state_dict is not None and template is not state_dict:
            for k, v in template.items():
                if k in state_dict:
                    state_dict[k].copy_(v)
        return self.current_version

    def get_transfer_stats(self) -> Dict:
        st = self.stats
        return {"backend": self.backend, "current_version": int(self.version), "total_syncs": st.sync_count,
                "last_transfer": {"total_params": st.total_params, "total_bytes": st.total_bytes,
                                  "total_bytes_human": f"{st.total_bytes / 1e9:.2f} GB",
                                  "broadcast_time_s": st.broadcast_time, "serialization_time_s": st.serialization_time,
                                  "total_time_s": st.total_time, "bandwidth_gbps": st.bandwidth_gbps},
                "history": list(st.history)}

    def get_stats(self) -> Dict:
        return {"backend": self.backend, "version": self.version, "transfers": self.stats.transfers,
                "total_bytes": self.stats.total_bytes, "avg_gbps": self.stats.avg_gbps,
                "failures": self.stats.failures}
