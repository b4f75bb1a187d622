"""Failure detection for multi-rank jobs: heartbeats, a step watchdog, typed errors.

The reference has only host-level safeguards (worker processes die with their parent, per-job
exceptions are reported through a queue, joins time out: reference ``tah/evaluate/jobs.py:310-358``,
``script/preparation/label.py:437-483``) and no elastic logic for training.  This module adds what
a long-running sharded job needs while staying on the host:

* :class:`RankHeartbeat` - every rank bumps a counter in the rendezvous store from a thread;
  :meth:`RankHeartbeat.check_peers` raises :class:`RankFailure` naming ranks whose counter stopped.
  Ranks call it between steps, i.e. *before* launching kernels that wait for a peer.
* :class:`StepWatchdog` - turns a step that exceeds its deadline into a :class:`StepTimeout` in the
  main thread (or a callback), so that a stalled collective becomes a clean abort + resume.
* device-side waits are bounded by construction (``csrc/common.cuh``); the host reads the status
  word with :func:`tah_b200.ops.cuda.check_status` and gets a :class:`~tah_b200.ops.cuda.KernelTimeout`.
"""
from __future__ import annotations

import threading
import time
from typing import Callable, List, Optional


class RankFailure(RuntimeError):
    def __init__(self, dead: List[int], message: str = ""):
        super().__init__(message or f"ranks {dead} stopped sending heartbeats")
        self.dead = dead


class StepTimeout(RuntimeError):
    pass


class RankHeartbeat:
    """``store`` is any object with ``set(key, value)`` / ``get(key)`` (a ``torch.distributed.TCPStore``,
    ``FileStore`` or a dict-backed fake in tests)."""

    def __init__(self, store, rank: int, world: int, interval_s: float = 0.5, prefix: str = "hb"):
        self.store, self.rank, self.world, self.interval, self.prefix = store, rank, world, interval_s, prefix
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self._count = 0
        self._seen = {}          # rank -> (last counter value, local time it last changed)

    def _key(self, r: int) -> str:
        return f"{self.prefix}/{r}"

    def beat(self) -> None:
        self._count += 1
        self.store.set(self._key(self.rank), str(self._count))

    def start(self) -> "RankHeartbeat":
        self.beat()

        def loop():
            while not self._stop.wait(self.interval):
                try:
                    self.beat()
                except Exception:
                    return
        self._thread = threading.Thread(target=loop, daemon=True)
        self._thread.start()
        return self

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2 * self.interval + 1)

    def check_peers(self, timeout_s: float = 5.0) -> None:
        """Raise :class:`RankFailure` if a peer's counter has not moved for ``timeout_s``."""
        now = time.monotonic()
        dead = []
        for r in range(self.world):
            if r == self.rank:
                continue
            try:
                val = self.store.get(self._key(r))
                val = val.decode() if isinstance(val, bytes) else str(val)
            except Exception:
                val = None
            last = self._seen.get(r)
            if last is None or last[0] != val:
                self._seen[r] = (val, now)
            elif now - last[1] > timeout_s:
                dead.append(r)
        if dead:
            raise RankFailure(dead)


class StepWatchdog:
    """``with StepWatchdog(30, on_timeout): step()`` - ``on_timeout`` runs in a helper thread when the
    body has not finished in time; without a callback the timeout is raised when the body returns."""

    def __init__(self, deadline_s: float, on_timeout: Optional[Callable[[], None]] = None):
        self.deadline, self.on_timeout = deadline_s, on_timeout
        self.fired = False
        self._done = threading.Event()

    def __enter__(self):
        def watch():
            if not self._done.wait(self.deadline):
                self.fired = True
                if self.on_timeout is not None:
                    self.on_timeout()
        threading.Thread(target=watch, daemon=True).start()
        return self

    def __exit__(self, exc_type, exc, tb):
        self._done.set()
        if self.fired and exc_type is None and self.on_timeout is None:
            raise StepTimeout(f"step exceeded its {self.deadline:.1f} s deadline")
        return False
