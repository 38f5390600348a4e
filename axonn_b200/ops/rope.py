"""Rotary position embedding, applied in place to ``[B, S, heads, D]`` tensors
(rotate-half convention, pairs ``(i, i + D/2)``; kernel in ``csrc/elementwise.cu``)."""

import ctypes

import torch

from . import _lib

_tables = {}


def rope_table(seq_len, head_dim, theta, device):
    """``[S, D/2, 2]`` fp32 table of (cos, sin)."""
    key = (seq_len, head_dim, float(theta), str(device))
    t = _tables.get(key)
    if t is None:
        inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float64) / head_dim))
        ang = torch.outer(torch.arange(seq_len, dtype=torch.float64), inv)
        t = torch.stack([ang.cos(), ang.sin()], -1).float().to(device).contiguous()
        _tables[key] = t
    return t


def _rope_torch(x, table, inverse, seq_dim=1):
    S, D = x.shape[seq_dim], x.shape[-1]
    shape = [1] * x.ndim
    shape[seq_dim], shape[-1] = S, D // 2
    cos = table[:S, :, 0].view(shape)
    sin = table[:S, :, 1].view(shape) * (-1.0 if inverse else 1.0)
    a, b = x[..., : D // 2].float(), x[..., D // 2:].float()
    return torch.cat([a * cos - b * sin, b * cos + a * sin], -1).to(x.dtype)


def _rope_apply(x, table, inverse):
    """x: ``[B, S, heads, D]`` or ``[B, S, groups, heads, D]`` (a view whose head/feature
    dims are dense and whose leading dims collapse to one row stride); rotated in
    place on GPU."""
    if not x.is_cuda:
        return _rope_torch(x, table, inverse)
    D, nh = x.shape[-1], x.shape[-2]
    S = x.shape[1]
    assert x.stride(-1) == 1 and x.stride(-2) == D and x.dtype == torch.bfloat16
    if x.ndim == 4:
        rows, pos_div, row_stride = x.shape[0] * S, 1, x.stride(1)
        assert x.stride(0) == S * x.stride(1), "batch and sequence dims must be collapsible"
    else:
        G = x.shape[2]
        rows, pos_div, row_stride = x.shape[0] * S * G, G, x.stride(2)
        assert x.stride(1) == G * x.stride(2) and x.stride(0) == S * x.stride(1)
    st = _lib.lib().axb_rope(_lib.ptr(x), _lib.ptr(table), ctypes.c_longlong(rows), ctypes.c_int(S),
                             ctypes.c_int(nh), ctypes.c_int(D), ctypes.c_int(pos_div),
                             ctypes.c_longlong(row_stride), ctypes.c_int(1 if inverse else 0), _lib.stream_ptr())
    _lib.check(st, "axb_rope")
    return x


class _RopeFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, table):
        ctx.table = table
        if x.is_cuda:
            ctx.mark_dirty(x)
        return _rope_apply(x, table, False)

    @staticmethod
    def backward(ctx, g):
        if g.is_cuda:
            g = g.contiguous() if not (g.stride(-1) == 1 and g.stride(-2) == g.shape[-1]) else g.clone()
        return _rope_apply(g, ctx.table, True), None


def apply_rope(x, table):
    """Rotate ``x`` (``[B, S, heads, D]`` or ``[B, S, groups, heads, D]``).  On GPU ``x``
    must be a non-leaf tensor (it is updated in place)."""
    return _RopeFn.apply(x, table)
