"""Multi-tensor utilities: squared L2 norm, in-place scale, bucketed all-reduce.

GPU paths use one launch over a table of tensor pointers
(``csrc/optim.cu``); they replace the per-tensor ``torch.norm`` stacks
and ``mul_`` loops of the reference's ``gradient_normalization.py:22-25,88-93``
and the per-tensor all-reduces of ``intra_layer/__init__.py:93-111,154-173``.
"""

import ctypes

import torch
import torch.distributed as dist

from . import _lib

_CHUNK = 1 << 16


_DT_CODE = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}


class _PtrTable:
    """Device table {pointer, numel, dtype, chunk prefix} for a list of tensors."""

    def __init__(self, tensors):
        dev = tensors[0].device
        rows, prefix = [], 0
        for t in tensors:
            assert t.is_contiguous(), "multi-tensor ops need contiguous tensors"
            rows.append((t.data_ptr(), t.numel(), _DT_CODE[t.dtype], prefix))
            prefix += (t.numel() + _CHUNK - 1) // _CHUNK
        self.n = len(rows)
        self.total_chunks = prefix
        self.host = torch.tensor(rows, dtype=torch.int64).pin_memory()
        self.dev = self.host.to(dev, non_blocking=True)
        self.keep = tensors


# Tables of recently used tensor lists, keyed by (pointer, numel, dtype) of every tensor: gradient lists
# repeat from step to step (the caching allocator hands the same blocks back), so the per-step utilities
# neither allocate pinned memory nor copy a table to the device after the first few steps.
_table_cache = {}
_TABLE_CACHE_MAX = 16


def _cached_table(tensors):
    key = tuple((t.data_ptr(), t.numel(), t.dtype) for t in tensors)
    tab = _table_cache.get(key)
    if tab is None:
        if len(_table_cache) >= _TABLE_CACHE_MAX:
            _table_cache.pop(next(iter(_table_cache)))
        tab = _PtrTable(tensors)
        tab.keep = None   # the cache must not keep gradient tensors alive
        _table_cache[key] = tab
    return tab


def multi_tensor_l2norm_sq(tensors):
    """sum_i ||t_i||_2^2 as a 0-d fp32 tensor on the tensors' device."""
    tensors = [t for t in tensors if t.numel() > 0]
    if not tensors:
        return torch.zeros((), dtype=torch.float32)
    if tensors[0].is_cuda:
        tab = _cached_table(tensors)
        out = torch.zeros((), dtype=torch.float32, device=tensors[0].device)
        st = _lib.lib().axb_multi_l2norm_sq(_lib.ptr(tab.dev), ctypes.c_int(tab.n),
                                            ctypes.c_longlong(tab.total_chunks), _lib.ptr(out), _lib.stream_ptr())
        _lib.check(st, "axb_multi_l2norm_sq")
        return out
    return torch.stack([t.detach().float().pow(2).sum() for t in tensors]).sum()


def multi_tensor_scale_(tensors, scale):
    """``t *= scale`` for every tensor; ``scale`` is a float or a 0-d tensor
    (kept on device: no host synchronisation)."""
    tensors = [t for t in tensors if t.numel() > 0]
    if not tensors:
        return
    if tensors[0].is_cuda:
        tab = _cached_table(tensors)
        if not torch.is_tensor(scale):
            scale = torch.full((), float(scale), dtype=torch.float32, device=tensors[0].device)   # no host sync
        else:
            scale = scale.to(device=tensors[0].device, dtype=torch.float32)
        st = _lib.lib().axb_multi_scale(_lib.ptr(tab.dev), ctypes.c_int(tab.n),
                                        ctypes.c_longlong(tab.total_chunks), _lib.ptr(scale), _lib.stream_ptr())
        _lib.check(st, "axb_multi_scale")
        return
    for t in tensors:
        t.mul_(scale.to(t.device) if torch.is_tensor(scale) else scale)


def all_reduce_bucketed_(grads, group, scale=None, coalesce=True, bucket_bytes=256 << 20):
    """Sum every tensor of ``grads`` over ``group`` in place, then multiply by
    ``scale``.  Tensors are packed into flat buckets (sized for launch latency,
    not link count: every peer is one NVSwitch hop away) so that a handful of
    collectives replace hundreds."""
    if not grads:
        return
    from ..parallel import fused

    if fused.try_all_reduce_scale_(grads, group, scale):
        return
    if not coalesce:
        for g in grads:
            dist.all_reduce(g, group=group)
            if scale is not None:
                g.mul_(scale)
        return
    by_dtype = {}
    for g in grads:
        by_dtype.setdefault(g.dtype, []).append(g)
    for dtype, gs in by_dtype.items():
        bucket, size = [], 0
        for g in gs + [None]:
            if g is not None and (size + g.numel() * g.element_size() <= bucket_bytes or not bucket):
                bucket.append(g)
                size += g.numel() * g.element_size()
                continue
            flat = torch._utils._flatten_dense_tensors(bucket)
            dist.all_reduce(flat, group=group)
            if scale is not None:
                flat.mul_(scale)
            for old, new in zip(bucket, torch._utils._unflatten_dense_tensors(flat, bucket)):
                old.copy_(new)
            bucket, size = ([g], g.numel() * g.element_size()) if g is not None else ([], 0)
