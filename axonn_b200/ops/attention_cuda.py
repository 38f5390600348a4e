"""Bindings of the flash-attention kernels (``csrc/flash_attn.cu``).

Forward and backward run on the package's tcgen05 kernels directly on the packed
QKV tensor (no split, no head repetition for grouped-query attention).
"""

import ctypes
import os

import torch

from . import _lib

_BWD_DEFAULT = "fused"


def available():
    return hasattr(_lib.lib(), "axb_flash_attn_fwd") and os.environ.get("AXONN_FLASH", "1") == "1"


def supported(qkv):
    B, S, G, n, D = qkv.shape
    return qkv.dtype == torch.bfloat16 and D in (64, 128) and S % 128 == 0 and qkv.is_contiguous()


def flash_fwd_packed(qkv, scale):
    """qkv [B, S, G, qpk+2, D] -> (out [B, S, G*qpk, D], lse [B, G*qpk, S])."""
    B, S, G, n, D = qkv.shape
    qpk = n - 2
    out = torch.empty((B, S, G * qpk, D), dtype=qkv.dtype, device=qkv.device)
    lse = torch.empty((B, G * qpk, S), dtype=torch.float32, device=qkv.device)
    st = _lib.lib().axb_flash_attn_fwd(_lib.ptr(qkv), _lib.ptr(out), _lib.ptr(lse), ctypes.c_int(B), ctypes.c_int(S),
                                       ctypes.c_int(G), ctypes.c_int(qpk), ctypes.c_int(D), ctypes.c_float(scale),
                                       ctypes.c_int(qkv.device.index), _lib.stream_ptr())
    _lib.check(st, "axb_flash_attn_fwd")
    return out, lse


def _bwd_split(qkv, out, d_out, lse, delta, dqkv, scale, which):
    B, S, G, n, D = qkv.shape
    st = _lib.lib().axb_flash_attn_bwd_split(
        _lib.ptr(qkv), _lib.ptr(out), _lib.ptr(d_out), _lib.ptr(lse), _lib.ptr(delta), _lib.ptr(dqkv),
        ctypes.c_int(B), ctypes.c_int(S), ctypes.c_int(G), ctypes.c_int(n - 2), ctypes.c_int(D),
        ctypes.c_float(scale), ctypes.c_int(which), ctypes.c_int(qkv.device.index), _lib.stream_ptr())
    _lib.check(st, "axb_flash_attn_bwd_split")
    _lib.add_launches(1)


def flash_bwd_packed(qkv, out, d_out, lse, scale):
    """Gradient of the packed QKV tensor for ``flash_fwd_packed``.

    ``AXONN_FA_BWD`` selects the implementation: ``split`` - the two-kernel backward without atomics
    (``csrc/flash_attn_bwd_split.cu``: one kernel for dQ, one for dK and dV); ``fused`` - the one-kernel form
    (``csrc/flash_attn.cu``) with its fp32 dQ accumulator; ``split_dq`` / ``split_dkv`` take only dQ or only
    dK, dV from the two-kernel form (A/B runs)."""
    B, S, G, n, D = qkv.shape
    qpk = n - 2
    H = G * qpk
    mode = os.environ.get("AXONN_FA_BWD", _BWD_DEFAULT)
    d_out = d_out if d_out.is_contiguous() else d_out.contiguous()
    delta = torch.empty((B, H, S), dtype=torch.float32, device=qkv.device)
    dqkv = torch.empty_like(qkv)
    if mode == "split":
        _bwd_split(qkv, out, d_out, lse, delta, dqkv, scale, 3)
        return dqkv
    dq_acc = torch.zeros((B, S, H, D), dtype=torch.float32, device=qkv.device)
    st = _lib.lib().axb_flash_attn_bwd(_lib.ptr(qkv), _lib.ptr(out), _lib.ptr(d_out), _lib.ptr(lse), _lib.ptr(delta),
                                       _lib.ptr(dq_acc), _lib.ptr(dqkv), ctypes.c_int(B), ctypes.c_int(S),
                                       ctypes.c_int(G), ctypes.c_int(qpk), ctypes.c_int(D), ctypes.c_float(scale),
                                       ctypes.c_int(qkv.device.index), _lib.stream_ptr())
    _lib.check(st, "axb_flash_attn_bwd")
    _lib.add_launches(1)
    dqkv[:, :, :, :qpk].copy_(dq_acc.view(B, S, G, qpk, D))
    if mode == "split_dq":
        _bwd_split(qkv, out, d_out, lse, delta, dqkv, scale, 1)
    elif mode == "split_dkv":
        _bwd_split(qkv, out, d_out, lse, delta, dqkv, scale, 2)
    return dqkv


class _FlashPacked(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, scale):
        out, lse = flash_fwd_packed(qkv, scale)
        ctx.save_for_backward(qkv, out, lse)
        ctx.scale = scale
        return out

    @staticmethod
    def backward(ctx, g):
        qkv, out, lse = ctx.saved_tensors
        return flash_bwd_packed(qkv, out, g, lse, ctx.scale), None


def flash_attention_packed_cuda(qkv, causal, scale):
    assert causal
    return _FlashPacked.apply(qkv, scale)
