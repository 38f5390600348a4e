"""Liveness watchdog: host-side failure detection for SPMD ranks.

The reference has no failure detection; a dead rank leaves its peers blocked
in a collective or in the pipeline's receive loop forever.  Here every rank
runs a daemon thread that publishes a heartbeat counter in the process group's
key-value store and watches its peers' counters.  When a peer's heartbeat has
not advanced for ``timeout_s`` the watchdog records the failure, invokes the
``on_failure`` callback (default: remember it so that ``check()`` raises
``RankFailure`` at the next step boundary) and can abort the process groups so
that blocked collectives return with an error.

Device-side waits are covered separately: every kernel of the package that
spins on a peer's flag has a deadline and reports through a status word
(``ops._lib.lib().axb_device_status``) instead of hanging the GPU.
"""

import threading
import time
from typing import Callable, Optional

import torch.distributed as dist


class RankFailure(RuntimeError):
    pass


class Watchdog:
    """Heartbeat thread of one rank: ``start()``, then ``check()`` at step boundaries (raises ``RankFailure`` naming
    the silent rank), ``stop()`` at the end.  ``store`` defaults to the default process group's store."""

    def __init__(self, store=None, rank: Optional[int] = None, world_size: Optional[int] = None,
                 interval_s: float = 0.5, timeout_s: float = 10.0,
                 on_failure: Optional[Callable[[int, float], None]] = None, prefix: str = "axonn_hb"):
        if store is None:
            store = dist.distributed_c10d._get_default_store()
        self.store = store
        self.rank = dist.get_rank() if rank is None else rank
        self.world = dist.get_world_size() if world_size is None else world_size
        self.interval_s, self.timeout_s = interval_s, timeout_s
        self.on_failure = on_failure
        self.prefix = prefix
        self.failed = {}
        self._stop = threading.Event()
        self._thread = None
        self._beat = 0

    def _key(self, r):
        return f"{self.prefix}/{r}"

    def start(self):
        self.store.set(self._key(self.rank), "0")
        self._thread = threading.Thread(target=self._run, daemon=True, name="axonn-watchdog")
        self._thread.start()
        return self

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2 * self.interval_s + 1)

    def _run(self):
        last_seen = {r: (None, time.monotonic()) for r in range(self.world) if r != self.rank}
        while not self._stop.is_set():
            self._beat += 1
            try:
                self.store.set(self._key(self.rank), str(self._beat))
            except Exception:
                return  # store gone: the job is shutting down
            now = time.monotonic()
            for r in list(last_seen):
                if r in self.failed:
                    continue
                try:
                    if not self.store.check([self._key(r)]):
                        val = None
                    else:
                        val = self.store.get(self._key(r)).decode()
                except Exception:
                    val = None
                prev, since = last_seen[r]
                if val is not None and val != prev:
                    last_seen[r] = (val, now)
                elif now - since > self.timeout_s:
                    self.failed[r] = now - since
                    if self.on_failure is not None:
                        self.on_failure(r, now - since)
            self._stop.wait(self.interval_s)

    def check(self):
        """Raise ``RankFailure`` if a peer has stopped responding (call between steps)."""
        if self.failed:
            r, silent = next(iter(self.failed.items()))
            raise RankFailure(f"rank {r} has not sent a heartbeat for {silent:.1f}s")
