"""Bindings of the flash-attention kernels (``csrc/flash_attn.cu``).

Forward runs on the package's tcgen05 kernel directly on the packed QKV
tensor; backward recomputes through ``F.scaled_dot_product_attention`` (cuDNN)
until the native backward kernel lands, which needs q/k/v split out of the
packed tensor.
"""

import ctypes
import os

import torch
import torch.nn.functional as F

from . import _lib


def available():
    return hasattr(_lib.lib(), "axb_flash_attn_fwd") and os.environ.get("AXONN_FLASH", "0") == "1"


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


class _FlashPacked(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, scale):
        out, lse = flash_fwd_packed(qkv, scale)
        ctx.save_for_backward(qkv)
        ctx.scale = scale
        return out

    @staticmethod
    def backward(ctx, g):
        (qkv,) = ctx.saved_tensors
        B, S, G, n, D = qkv.shape
        qpk = n - 2
        with torch.enable_grad():
            x = qkv.detach().requires_grad_(True)
            q = x[:, :, :, :qpk].reshape(B, S, G * qpk, D).transpose(1, 2)
            k = x[:, :, :, qpk].transpose(1, 2).repeat_interleave(qpk, dim=1)
            v = x[:, :, :, qpk + 1].transpose(1, 2).repeat_interleave(qpk, dim=1)
            o = F.scaled_dot_product_attention(q, k, v, is_causal=True, scale=ctx.scale).transpose(1, 2)
            (gx,) = torch.autograd.grad(o, x, g)
        return gx, None


def flash_attention_packed_cuda(qkv, causal, scale):
    assert causal
    return _FlashPacked.apply(qkv, scale)
