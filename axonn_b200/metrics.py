"""Throughput, MFU and memory accounting with a JSONL sink.

The reference prints loss and peak memory from its (stale) example scripts
only (``examples/test_lm.py:118-124,245-252``); this module is the structured
replacement used by ``bench.py`` and the training entry points: every step is
timed on the device (CUDA events), reduced with MAX over ranks, and turned
into tokens/s and model-FLOPs utilisation against the measured bf16 peak.
"""

import json
import os
import time
from typing import Optional

import torch
import torch.distributed as dist

_FALLBACK_PEAK_TFLOPS = 1400.0


def measured_peaks(path: Optional[str] = None):
    """(bf16 sustained TFLOP/s, HBM GB/s, 'measured' | 'fallback')."""
    here = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    path = path or os.environ.get("AXONN_MEASURED_PEAKS", os.path.join(here, "MEASURED_PEAKS.json"))
    try:
        with open(path) as f:
            d = json.load(f)
        return float(d["bf16_tflops_sustained"]), float(d["hbm_gbs"]), "measured"
    except Exception:
        return _FALLBACK_PEAK_TFLOPS, 6650.0, "fallback"


class StepMeter:
    """Device-timed step statistics.

    with meter.step(tokens): ... one training step ...
    meter.summary() -> dict(tokens_per_s, ms_per_step, mfu, peak_mem_gb)"""

    def __init__(self, flops_per_token: float = 0.0, world_size: Optional[int] = None, log_path: Optional[str] = None):
        self.flops_per_token = flops_per_token
        self.world = world_size or (dist.get_world_size() if dist.is_initialized() else 1)
        self.log_path = log_path
        self.records = []
        self.use_cuda = torch.cuda.is_available()
        self.peak_tflops, _, self.peak_kind = measured_peaks()

    class _Ctx:
        def __init__(self, meter, tokens):
            self.m, self.tokens = meter, tokens

        def __enter__(self):
            if self.m.use_cuda:
                self.e0 = torch.cuda.Event(enable_timing=True)
                self.e1 = torch.cuda.Event(enable_timing=True)
                self.e0.record()
            else:
                self.t0 = time.perf_counter()
            return self

        def __exit__(self, *exc):
            if self.m.use_cuda:
                self.e1.record()
                self.m.records.append((self.tokens, (self.e0, self.e1)))
            else:
                self.m.records.append((self.tokens, (time.perf_counter() - self.t0) * 1e3))
            return False

    def step(self, global_tokens: int):
        return StepMeter._Ctx(self, global_tokens)

    def summary(self, reset=True):
        if self.use_cuda:
            torch.cuda.synchronize()
        ms = [(r[1][0].elapsed_time(r[1][1]) if self.use_cuda else r[1]) for r in self.records]
        tokens = sum(r[0] for r in self.records)
        total = torch.tensor([sum(ms)], dtype=torch.float64, device="cuda" if self.use_cuda else "cpu")
        if dist.is_initialized() and dist.get_world_size() > 1:
            dist.all_reduce(total, op=dist.ReduceOp.MAX)
        total_ms = float(total.item())
        n = max(1, len(ms))
        out = {
            "steps": len(ms), "ms_per_step": total_ms / n,
            "tokens_per_s": tokens / (total_ms / 1e3) if total_ms > 0 else 0.0,
            "mfu": (self.flops_per_token * tokens / (total_ms / 1e3) / (self.world * self.peak_tflops * 1e12)
                    if total_ms > 0 and self.flops_per_token else None),
            "mfu_peak_tflops": self.peak_tflops, "mfu_peak_kind": self.peak_kind,
            "peak_mem_gb": torch.cuda.max_memory_allocated() / 2 ** 30 if self.use_cuda else None,
        }
        if self.log_path and (not dist.is_initialized() or dist.get_rank() == 0):
            with open(self.log_path, "a") as f:
                f.write(json.dumps(out) + "\n")
        if reset:
            self.records = []
        return out


# ----------------------------------------------------------------------------- exposed communication
# Kernel names that only move data between ranks (a collective library's kernels and this package's
# stand-alone peer-memory kernels).  Fused compute+collective kernels are compute kernels here; the time
# they spend waiting on peers is counted inside the kernels (``fused_comm_stall_ms``).
COMM_KERNEL_PATTERNS = ("nccl", "allreduce_twoshot", "grad_allreduce", "bucket_copy", "moe_scatter_rows", "moe_gather_rows",
                        "moe_signal", "moe_wait", "a2a_v", "embedding_p2p", "symm_all_gather", "symm_reduce_scatter")


def is_comm_kernel(name: str) -> bool:
    """True for kernels whose time counts as communication in the exposed-communication figure (NCCL kernels
    and this package's stand-alone peer-memory collectives)."""
    low = name.lower()
    return any(p in low for p in COMM_KERNEL_PATTERNS)


def _union(intervals):
    """Merge [(start, end), ...] into disjoint sorted intervals."""
    out = []
    for s, e in sorted(intervals):
        if e <= s:
            continue
        if out and s <= out[-1][1]:
            if e > out[-1][1]:
                out[-1][1] = e
        else:
            out.append([s, e])
    return out


def _length(intervals):
    return sum(e - s for s, e in intervals)


def _subtract(a, b):
    """Parts of the disjoint sorted intervals ``a`` not covered by the disjoint sorted intervals ``b``."""
    out, j = [], 0
    for s, e in a:
        cur = s
        while j < len(b) and b[j][1] <= cur:
            j += 1
        k = j
        while k < len(b) and b[k][0] < e:
            if b[k][0] > cur:
                out.append([cur, min(b[k][0], e)])
            cur = max(cur, b[k][1])
            if cur >= e:
                break
            k += 1
        if cur < e:
            out.append([cur, e])
    return out


def exposed_comm_from_intervals(kernels):
    """``kernels``: iterable of (name, start, end) device intervals of one rank (any unit).  Returns
    (exposed, comm_total, compute_total): the time during which a communication kernel runs and no compute
    kernel does (union of the communication intervals minus the union of the compute intervals), the union
    of the communication intervals and the union of the compute intervals.  This is the part of the
    communication that the step pays for; the reference's exposed points are its blocking forward
    all-reduce (``axonn/intra_layer/fully_connected.py:119``) and the device-wide synchronisation that ends
    every overlap window (``axonn/intra_layer/overlap_communication.py:27-30``)."""
    comm, comp = [], []
    for name, s, e in kernels:
        (comm if is_comm_kernel(name) else comp).append((s, e))
    comm_u, comp_u = _union(comm), _union(comp)
    return _length(_subtract(comm_u, comp_u)), _length(comm_u), _length(comp_u)


def profile_exposed_comm(step_fn, fused_stall=True):
    """Run ``step_fn()`` once under the PyTorch profiler (device activities only) and account its kernels.
    Returns a dict with ``exposed_comm_ms`` (communication kernels not covered by compute kernels),
    ``comm_kernel_ms``, ``compute_kernel_ms`` and, for this package's fused kernels,
    ``fused_comm_stall_ms``: the mean per-CTA time that the fused GEMM kernels of the step spent waiting
    for peers (weight shards not yet arrived + the tail after the CTA's last tile in which only the
    reduction of peer data remained), measured inside the kernels with the global timer."""
    from torch.profiler import ProfilerActivity, profile

    if fused_stall:
        fused_comm_stall(reset=True)
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        step_fn()
        torch.cuda.synchronize()
    kernels = []
    for ev in prof.events():
        if getattr(ev, "device_type", None) is not None and "cuda" in str(ev.device_type).lower():
            tr = ev.time_range
            kernels.append((ev.name, float(tr.start), float(tr.end)))
    exposed, comm, comp = exposed_comm_from_intervals(kernels)
    stall = fused_comm_stall(reset=True) if fused_stall else 0.0
    return {"exposed_comm_ms": exposed / 1e3, "comm_kernel_ms": comm / 1e3, "compute_kernel_ms": comp / 1e3,
            "fused_comm_stall_ms": stall, "kernels": len(kernels)}


def fused_comm_stall(reset=True) -> float:
    """Milliseconds that the fused GEMM kernels launched since the last reset spent stalled on peers, as the
    sum over kernels of the mean over each kernel's CTAs (the CTAs of a kernel stall concurrently).  Zero when
    the native library is absent or no GPU is present."""
    try:
        import ctypes

        from .ops import _lib

        if not (_lib.available() and torch.cuda.is_available()):
            return 0.0
        L = _lib.lib()
        L.axb_comm_stall_ms.restype = ctypes.c_double
        return float(L.axb_comm_stall_ms(ctypes.c_int(torch.cuda.current_device()), ctypes.c_int(1 if reset else 0)))
    except Exception:  # noqa: BLE001
        return 0.0
