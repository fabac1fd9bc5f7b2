"""Host-side failure detection for multi-rank jobs: heartbeats over the rendezvous store.

A rank that dies or stalls must surface on its peers as an exception on the HOST, before they launch kernels that would wait
for it. Every rank runs a ``PeerMonitor``: a daemon thread advances ``hb/<rank>`` in a ``torch.distributed`` store every
``interval`` seconds; ``check()`` (called by the training loop between steps) reads all counters and raises ``PeerLostError``
when a peer's counter has not moved for ``timeout`` seconds, unless that peer announced a clean exit with ``leave()``.
Device-side waits are bounded independently (``RECIS_WAIT_TIMEOUT_S``), so even without the monitor a missing peer ends a
step with an error status instead of a hang; the monitor turns that into a prompt, attributable error.

The reference relies on the 1800 s NCCL timeout only (``recis/framework/trainer.py:171``) and on a cooperative
end-of-data all-reduce (``trainer.py:346-349``).
"""
from __future__ import annotations

import threading
import time
from datetime import timedelta
from typing import Optional

import torch.distributed as dist


class PeerLostError(RuntimeError):
    def __init__(self, rank: int, silent_for: float):
        super().__init__(f"rank {rank} has not sent a heartbeat for {silent_for:.1f} s (crashed or stalled)")
        self.rank = rank


class PeerMonitor:
    def __init__(self, rank: int, world: int, store=None, interval: float = 0.5, timeout: float = 10.0, prefix: str = "recis_b200",
                 startup_timeout: Optional[float] = None):
        self.rank, self.world = rank, world
        self.interval, self.timeout, self.prefix = interval, timeout, prefix
        # ranks do not start their monitors at the same moment (imports, model construction): a peer that has not published
        # its first heartbeat yet is given this long before it counts as lost
        self.startup_timeout = max(60.0, 10 * timeout) if startup_timeout is None else startup_timeout
        self.store = store if store is not None else self._default_store()
        self._beat = 0
        self._stop = threading.Event()
        self._created = time.monotonic()
        self._last = {r: None for r in range(world)}          # (beat, time it last changed); None until the peer was first seen
        self._left = set()
        self._thread: Optional[threading.Thread] = None
        self._last_check = -1e30

    @staticmethod
    def _default_store():
        # the store of the default process group (TCPStore behind env:// rendezvous)
        return dist.distributed_c10d._get_default_store()

    def _key(self, kind: str, r: int) -> str:
        return f"{self.prefix}/{kind}/{r}"

    def start(self):
        self.store.set(self._key("hb", self.rank), "0")
        self._thread = threading.Thread(target=self._run, name="recis-heartbeat", daemon=True)
        self._thread.start()
        return self

    def _run(self):
        while not self._stop.wait(self.interval):
            self._beat += 1
            try:
                self.store.set(self._key("hb", self.rank), str(self._beat))
            except Exception:          # noqa: BLE001 - the store host went away: nothing left to report to
                return

    def pause(self):
        """Stop sending heartbeats without announcing an exit (what a hung process looks like; used by tests)."""
        self._stop.set()

    def leave(self):
        """Announce a clean exit: peers stop expecting heartbeats from this rank."""
        self._stop.set()
        try:
            self.store.set(self._key("left", self.rank), "1")
        except Exception:              # noqa: BLE001
            pass

    def check(self):
        """Raise ``PeerLostError`` if a peer that has not left went silent for longer than ``timeout``. The store is asked at
        most once per heartbeat interval (heartbeats cannot change faster), so calling this every step costs nothing between."""
        now = time.monotonic()
        if now - self._last_check < self.interval:
            return
        self._last_check = now
        for r in range(self.world):
            if r == self.rank or r in self._left:
                continue
            try:
                if self.store.check([self._key("left", r)]):
                    self._left.add(r)
                    continue
                beat = int(self.store.get(self._key("hb", r))) if self.store.check([self._key("hb", r)]) else None
            except Exception as e:     # noqa: BLE001 - the store itself is gone (rank 0 hosts it)
                raise PeerLostError(0, self.timeout) from e
            if beat is None:           # the peer's monitor has not started yet
                if now - self._created > self.startup_timeout:
                    raise PeerLostError(r, now - self._created)
                continue
            if self._last[r] is None:  # first sight: its clock starts now
                self._last[r] = (beat, now)
                continue
            last_beat, last_time = self._last[r]
            if beat != last_beat:
                self._last[r] = (beat, now)
            elif now - last_time > self.timeout:
                raise PeerLostError(r, now - last_time)

    def alive(self):
        return [r for r in range(self.world) if r not in self._left]


def init_process_group_with_timeout(backend: str, timeout_s: float, **kw):
    """``dist.init_process_group`` with a short collective timeout: a collective that a dead peer never joins raises after
    ``timeout_s`` seconds instead of blocking for the default half hour."""
    return dist.init_process_group(backend, timeout=timedelta(seconds=timeout_s), **kw)
