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
