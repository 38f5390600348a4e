"""GELU (tanh form) and SwiGLU (``csrc/elementwise.cu``)."""

import ctypes

import torch
import torch.nn.functional as F

from . import _lib


class _GeluFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        ctx.save_for_backward(x)
        if x.is_cuda and x.dtype == torch.bfloat16 and x.numel() % 8 == 0:
            x = x.contiguous()
            y = torch.empty_like(x)
            _lib.check(_lib.lib().axb_gelu_fwd(_lib.ptr(x), _lib.ptr(y), ctypes.c_longlong(x.numel()),
                                               _lib.stream_ptr()), "axb_gelu_fwd")
            return y
        if x.is_cuda:
            raise TypeError("gelu kernel needs bf16 input with numel % 8 == 0")
        return F.gelu(x, approximate="tanh")

    @staticmethod
    def backward(ctx, dy):
        (x,) = ctx.saved_tensors
        return gelu_backward(dy, x)


def gelu_backward_colsum(dy, x, out_dtype=torch.float32):
    """``dx = dy * gelu'(x)`` and ``dx.sum(0)`` (fp32 accumulation, returned as ``out_dtype``) of 2-D tensors in
    one pass: the backward of a fused bias + GELU layer needs both, and the column sums come for free while
    ``dx`` is being written."""
    if (x.is_cuda and x.dim() == 2 and x.shape[1] % 8 == 0 and x.dtype in (torch.bfloat16, torch.float16)
            and dy.dtype == x.dtype and x.shape[0] > 0):
        x, dy = x.contiguous(), dy.contiguous()
        rows, n = x.shape
        L = _lib.lib()
        dev = x.device.index
        splits = L.axb_colsum_splits(ctypes.c_int(dev), ctypes.c_int(rows), ctypes.c_int(n))
        part = torch.empty((splits, n), dtype=torch.float32, device=x.device)
        colsum = torch.empty(n, dtype=out_dtype, device=x.device)
        dx = torch.empty_like(x)
        _lib.check(L.axb_gelu_bwd_colsum(_lib.ptr(dy), _lib.ptr(x), _lib.ptr(dx), _lib.ptr(part), _lib.ptr(colsum),
                                         ctypes.c_int(rows), ctypes.c_int(n),
                                         ctypes.c_int(0 if x.dtype == torch.bfloat16 else 1),
                                         ctypes.c_int({torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}[out_dtype]),
                                         ctypes.c_int(dev), _lib.stream_ptr()), "axb_gelu_bwd_colsum")
        _lib.add_launches(1)
        return dx, colsum
    dx = gelu_backward(dy, x)
    return dx, dx.sum(0, dtype=torch.float32).to(out_dtype)


def gelu_backward(dy, x):
    """``dy * gelu'(x)`` (also used by the fused GEMM+GELU layer)."""
    if x.is_cuda:
        x, dy = x.contiguous(), dy.contiguous()
        dx = torch.empty_like(x)
        _lib.check(_lib.lib().axb_gelu_bwd(_lib.ptr(dy), _lib.ptr(x), _lib.ptr(dx),
                                           ctypes.c_longlong(x.numel()), _lib.stream_ptr()), "axb_gelu_bwd")
        return dx
    xf = x.float()
    k0, k1 = 0.7978845608028654, 0.044715
    u = k0 * (xf + k1 * xf ** 3)
    t = torch.tanh(u)
    d = 0.5 * (1 + t) + 0.5 * xf * (1 - t * t) * k0 * (1 + 3 * k1 * xf * xf)
    return (dy.float() * d).to(dy.dtype)


def gelu(x):
    """GELU (tanh form) with its backward as one kernel each."""
    return _GeluFn.apply(x)


class _SwiGLUFn(torch.autograd.Function):
    """``silu(gate) * up``; gate and up are interleaved in blocks of 8 along the last
    dim of ``gu`` (columns ``[16i, 16i+8)`` gate, ``[16i+8, 16i+16)`` up), which keeps
    the layout independent of how the fused projection is sharded."""

    @staticmethod
    def forward(ctx, gu):
        ctx.save_for_backward(gu)
        F2 = gu.shape[-1]
        Fh = F2 // 2
        if gu.is_cuda:
            if gu.dtype != torch.bfloat16 or Fh % 8:
                raise TypeError("swiglu kernel needs bf16 input with F % 8 == 0")
            g2 = gu.reshape(-1, F2).contiguous()
            out = torch.empty((g2.shape[0], Fh), dtype=gu.dtype, device=gu.device)
            _lib.check(_lib.lib().axb_swiglu_fwd(_lib.ptr(g2), _lib.ptr(out), ctypes.c_int(g2.shape[0]),
                                                 ctypes.c_int(Fh), _lib.stream_ptr()), "axb_swiglu_fwd")
            return out.reshape(*gu.shape[:-1], Fh)
        g, u = _split_gu(gu)
        return F.silu(g) * u

    @staticmethod
    def backward(ctx, dout):
        (gu,) = ctx.saved_tensors
        F2 = gu.shape[-1]
        Fh = F2 // 2
        if gu.is_cuda:
            g2 = gu.reshape(-1, F2).contiguous()
            d2 = dout.reshape(-1, Fh).contiguous()
            dgu = torch.empty_like(g2)
            _lib.check(_lib.lib().axb_swiglu_bwd(_lib.ptr(d2), _lib.ptr(g2), _lib.ptr(dgu),
                                                 ctypes.c_int(g2.shape[0]), ctypes.c_int(Fh),
                                                 _lib.stream_ptr()), "axb_swiglu_bwd")
            return dgu.reshape(gu.shape)
        g, u = (t.float() for t in _split_gu(gu))
        s = torch.sigmoid(g)
        silu = g * s
        d = dout.float()
        dg, du = d * u * (s + silu * (1 - s)), d * silu
        lead = gu.shape[:-1]
        out = torch.stack([dg.reshape(*lead, Fh // 8, 8), du.reshape(*lead, Fh // 8, 8)], -2)
        return out.reshape(gu.shape).to(gu.dtype)


def _split_gu(gu):
    F2 = gu.shape[-1]
    v = gu.reshape(*gu.shape[:-1], F2 // 16, 2, 8)
    return v[..., 0, :].reshape(*gu.shape[:-1], F2 // 2), v[..., 1, :].reshape(*gu.shape[:-1], F2 // 2)


def swiglu(gu):
    """``silu(gate) * up`` of a fused ``[..., 2 * ffn]`` projection whose gate and up columns alternate in blocks
    of 8 (the layout the fused gate|up weight of ``ParallelMLP`` produces); returns ``[..., ffn]``."""
    return _SwiGLUFn.apply(gu)
