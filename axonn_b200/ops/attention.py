"""Causal multi-head / grouped-query attention.

``flash_attention(q, k, v)`` takes ``[B, S, heads, D]`` tensors (``k``/``v`` may
have fewer heads: grouped-query attention).  ``flash_attention_packed(qkv)``
takes the fused projection output ``[B, S, G, q_per_kv + 2, D]`` — per KV group
its query heads, then its key head, then its value head — and avoids splitting
it.  Both return ``[B, S, heads, D]``.
"""

import math

import torch
import torch.nn.functional as F

_IMPL = {"force_torch": False}


def _sdpa(q, k, v, causal, scale):
    # [B, S, h, D] -> [B, h, S, D]
    qh, kh, vh = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
    rep = qh.shape[1] // kh.shape[1]
    if rep > 1:
        kh = kh.repeat_interleave(rep, dim=1)
        vh = vh.repeat_interleave(rep, dim=1)
    o = F.scaled_dot_product_attention(qh, kh, vh, is_causal=causal, scale=scale)
    return o.transpose(1, 2)


def flash_attention(q, k, v, causal=True, scale=None):
    """Attention of ``q [B, S, heads, D]`` against ``k, v [B, S, kv_heads, D]`` (grouped-query when ``kv_heads <
    heads``) on the package's tcgen05 kernels (CUDA, D 64 or 128, S a multiple of 128) or through
    ``scaled_dot_product_attention`` otherwise; returns ``[B, S, heads, D]``."""
    if scale is None:
        scale = 1.0 / math.sqrt(q.shape[-1])
    if q.is_cuda and not _IMPL["force_torch"]:
        from . import attention_cuda

        if attention_cuda.available() and causal:
            B, S, hq, D = q.shape
            G = k.shape[2]
            qkv = torch.cat([q.reshape(B, S, G, hq // G, D), k.unsqueeze(3), v.unsqueeze(3)], 3)
            if attention_cuda.supported(qkv):
                return attention_cuda.flash_attention_packed_cuda(qkv, causal, scale)
    return _sdpa(q, k, v, causal, scale)


def flash_attention_packed(qkv, causal=True, scale=None):
    """Attention on the packed projection output ``[B, S, kv_groups, q_per_kv + 2, D]`` (per KV group: its query
    heads, then K, then V) without splitting it into three tensors; returns ``[B, S, kv_groups * q_per_kv, D]``."""
    B, S, G, n, D = qkv.shape
    qpk = n - 2
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    if qkv.is_cuda and not _IMPL["force_torch"]:
        from . import attention_cuda

        if attention_cuda.available() and attention_cuda.supported(qkv) and causal:
            return attention_cuda.flash_attention_packed_cuda(qkv, causal, scale)
    q = qkv[:, :, :, :qpk].reshape(B, S, G * qpk, D)
    return _sdpa(q, qkv[:, :, :, qpk], qkv[:, :, :, qpk + 1], causal, scale)
