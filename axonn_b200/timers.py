"""Nested region timers.

Same user-facing contract as the reference's ``axonn/timers.py:7-46``
(``start``/``stop``/``get_times`` with stack-scoped keys, no-op unless enabled)
but the clock is chosen per device: CUDA events on the current stream when a
GPU is in use, ``time.perf_counter`` on CPU, so the whole API also works under
gloo.  Regions additionally emit NVTX ranges when CUDA is available.
"""

import time
from collections import defaultdict

import torch


class _CpuStamp:
    __slots__ = ("t",)

    def __init__(self):
        self.t = None

    def record(self):
        self.t = time.perf_counter()

    def elapsed_time(self, other):
        return (other.t - self.t) * 1e3


class Timers:
    """Nested region timers (reference ``axonn/timers.py:7-46``): ``start(key)`` / ``stop(key)`` pairs may nest,
    and a region is accounted under the tuple of all keys open at that moment, so the same inner key under two
    different parents gives two series.  Times come from CUDA events on GPUs (no host synchronisation until
    ``get_times``) and from ``perf_counter`` on CPU; every region is also an NVTX range."""

    def __init__(self, enabled=True, use_cuda=None, nvtx=True):
        self.enabled = enabled
        self.use_cuda = torch.cuda.is_available() if use_cuda is None else use_cuda
        self.nvtx = nvtx and self.use_cuda
        self.stack = []
        self.events = defaultdict(list)  # key tuple -> [(start, stop), ...]
        self.open = {}

    def _stamp(self):
        if self.use_cuda:
            ev = torch.cuda.Event(enable_timing=True)
        else:
            ev = _CpuStamp()
        ev.record()
        return ev

    def start(self, key):
        if not self.enabled:
            return
        self.stack.append(key)
        k = tuple(self.stack)
        if self.nvtx:
            torch.cuda.nvtx.range_push(str(key))
        self.open[k] = self._stamp()

    def stop(self, key):
        if not self.enabled:
            return
        k = tuple(self.stack)
        assert self.stack and self.stack[-1] == key, (
            f"timer stop({key!r}) does not match innermost start "
            f"({self.stack[-1] if self.stack else None!r})"
        )
        stop = self._stamp()
        if self.nvtx:
            torch.cuda.nvtx.range_pop()
        self.events[k].append((self.open.pop(k), stop))
        self.stack.pop()

    def get_times(self):
        """Return ``(total_ms, counts)`` keyed by the nested key tuple and reset."""
        if self.use_cuda:
            torch.cuda.synchronize()
        total, counts = {}, {}
        for k, pairs in self.events.items():
            total[k] = sum(a.elapsed_time(b) for a, b in pairs)
            counts[k] = len(pairs)
        self.events = defaultdict(list)
        return total, counts


class _NullTimers(Timers):
    """Disabled timers: every call is a no-op."""

    def __init__(self):
        super().__init__(enabled=False, use_cuda=False, nvtx=False)
