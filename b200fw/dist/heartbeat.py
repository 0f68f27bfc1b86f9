"""Host-side liveness of the ranks of a job, over the rendezvous key-value store.

A rank that has gone (crashed, killed, left on an error) is otherwise noticed only when a collective that needs it
times out, or - on the peer-memory data plane - when a kernel's bounded wait for that rank's flag runs out.  Both
come late and after work was launched.  Here every rank bumps a counter in the store from a daemon thread and watches
its peers' counters; a peer whose counter stands still for ``timeout_s``, or that announced its leave, marks the
watcher as ``lost``, and :meth:`RankHeartbeat.check` - a local read, free to call before every step - raises
:class:`PeerLostError` *before* the next kernel or collective is launched.

The reference has no such component: its only hang detection is the polling timeout of an asynchronous collective
handle (src/distributed/comm.py:313-352).  The store is the one ``torch.distributed`` already keeps for the process
group (``TCPStore`` behind ``env://``), so no extra port or service is needed; any c10d ``Store`` works (tests use
``HashStore`` and the gloo group's store).
"""
from __future__ import annotations

import threading
import time
from typing import Dict, Optional

from ..obs.logging import get_logger

logger = get_logger("dist.heartbeat")


class PeerLostError(RuntimeError):
    """A peer rank stopped answering (or said it leaves).  ``rank`` is the peer, ``reason`` what is known."""

    def __init__(self, rank: int, reason: str):
        super().__init__(f"rank {rank} is gone: {reason}")
        self.rank, self.reason = rank, reason


class RankHeartbeat:
    def __init__(self, store, rank: int, world_size: int, interval_s: float = 1.0, timeout_s: float = 10.0,
                 prefix: str = "b200fw/hb"):
        assert timeout_s > interval_s > 0
        self.store, self.rank, self.world = store, rank, world_size
        self.interval_s, self.timeout_s, self.prefix = interval_s, timeout_s, prefix
        self.lost: Optional[PeerLostError] = None
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self._seen: Dict[int, tuple] = {}           # peer -> (last counter value, local time it last changed)
        self.beats = 0

    # ---- construction ------------------------------------------------------------------------------------------------
    @classmethod
    def from_default_group(cls, interval_s: float = 1.0, timeout_s: float = 10.0) -> Optional["RankHeartbeat"]:
        """On the store of the default process group; ``None`` when there is no group or it keeps no store."""
        import torch.distributed as dist
        if not dist.is_available() or not dist.is_initialized() or dist.get_world_size() <= 1:
            return None
        try:
            store = dist.distributed_c10d._get_default_store()
        except Exception:  # noqa: BLE001 - a private accessor: absent or changed means "not available"
            return None
        return cls(store, dist.get_rank(), dist.get_world_size(), interval_s, timeout_s)

    # ---- keys -------------------------------------------------------------------------------------------------------
    def _beat_key(self, r: int) -> str:
        return f"{self.prefix}/beat/{r}"

    def _left_key(self, r: int) -> str:
        return f"{self.prefix}/left/{r}"

    # ---- the watcher thread --------------------------------------------------------------------------------------------
    def start(self) -> "RankHeartbeat":
        if self._thread is None:
            self.beat()                              # visible before anybody looks
            self._thread = threading.Thread(target=self._loop, name="b200fw-heartbeat", daemon=True)
            self._thread.start()
        return self

    def _loop(self):
        while not self._stop.wait(self.interval_s):
            try:
                self.beat()
                self.poll()
            except Exception as e:  # noqa: BLE001 - the store no longer answers: rank 0, which hosts it, is gone
                if self.lost is None and not self._stop.is_set():
                    self.lost = PeerLostError(0, f"the rendezvous store stopped answering ({type(e).__name__}: {e})")
                return

    def beat(self):
        self.store.add(self._beat_key(self.rank), 1)
        self.beats += 1

    def poll(self, now: Optional[float] = None):
        """One look at every peer (the thread calls this every interval; tests call it with their own clock)."""
        now = time.monotonic() if now is None else now
        for r in range(self.world):
            if r == self.rank or self.lost is not None:
                continue
            if self.store.check([self._left_key(r)]):
                self.lost = PeerLostError(r, "it announced its leave: " + self.store.get(self._left_key(r)).decode())
                break
            value = int(self.store.add(self._beat_key(r), 0))          # add 0: a read that never blocks on a missing key
            last = self._seen.get(r)
            if last is None or value != last[0]:
                self._seen[r] = (value, now)
            elif now - last[1] > self.timeout_s:
                self.lost = PeerLostError(r, f"no heartbeat for {now - last[1]:.1f} s (limit {self.timeout_s:.1f} s)")
                break
        if self.lost is not None:
            logger.error("%s", self.lost)

    # ---- what the training loop calls ------------------------------------------------------------------------------------
    def check(self):
        """Raise :class:`PeerLostError` if the watcher has found a peer gone.  A local read."""
        if self.lost is not None:
            raise self.lost

    def announce_leave(self, reason: str = "finished"):
        """Tell the peers that this rank leaves on purpose (between steps, nothing of it in flight), and stop."""
        try:
            self.store.set(self._left_key(self.rank), reason)
        except Exception:  # noqa: BLE001 - the store may be gone already at teardown
            pass
        self.stop()

    def stop(self):
        self._stop.set()
        t, self._thread = self._thread, None
        if t is not None and t is not threading.current_thread():
            t.join(timeout=2 * self.interval_s + 1)
