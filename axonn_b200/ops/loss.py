"""Softmax cross-entropy on (optionally vocabulary-parallel) logits.

The GPU path reads the bf16 logits once for the row statistics and rewrites
them in place with the gradient in backward, so no fp32 copy of the
``[tokens, vocab]`` matrix is ever materialised (``csrc/loss.cu``).
"""

import ctypes

import torch
import torch.distributed as dist

from . import _lib


class _CrossEntropyFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, targets, group, ignore_index):
        V = logits.shape[-1]
        z = logits.reshape(-1, V)
        t = targets.reshape(-1).contiguous()
        rows = z.shape[0]
        n = 1 if group is None else dist.get_world_size(group)
        start = 0 if n == 1 else dist.get_rank(group) * V
        if z.is_cuda:
            if z.dtype != torch.bfloat16:
                raise TypeError("cross-entropy kernel needs bf16 logits")
            z = z.contiguous()
            stats = torch.empty((rows, 3), dtype=torch.float32, device=z.device)
            _lib.check(_lib.lib().axb_ce_fwd(_lib.ptr(z), _lib.ptr(t), _lib.ptr(stats), ctypes.c_int(rows),
                                             ctypes.c_int(V), ctypes.c_int(start), _lib.stream_ptr()), "axb_ce_fwd")
            m, s, tl = stats[:, 0], stats[:, 1], stats[:, 2]
        else:
            zf = z.float()
            m = zf.max(-1).values
            s = (zf - m[:, None]).exp().sum(-1)
            loc = t - start
            inside = (loc >= 0) & (loc < V)
            tl = torch.where(inside, zf.gather(1, loc.clamp(0, V - 1)[:, None])[:, 0], torch.zeros_like(m))
        if n > 1:
            gm = m.clone()
            dist.all_reduce(gm, op=dist.ReduceOp.MAX, group=group)
            st = torch.stack([s * (m - gm).exp(), tl])
            dist.all_reduce(st, group=group)
            s, tl, m = st[0], st[1], gm
        lse = m + s.log()
        valid = t != ignore_index
        count = valid.sum().clamp_min(1).float()
        loss = ((lse - tl) * valid).sum() / count
        ctx.save_for_backward(z, t, lse.contiguous(), count)
        ctx.start, ctx.ignore_index, ctx.shape = start, ignore_index, logits.shape
        return loss

    @staticmethod
    def backward(ctx, g):
        z, t, lse, count = ctx.saved_tensors
        V = z.shape[-1]
        scale = (g.float() / count).reshape(1).contiguous()
        if z.is_cuda:
            _lib.check(_lib.lib().axb_ce_bwd(_lib.ptr(z), _lib.ptr(t), _lib.ptr(lse), _lib.ptr(scale),
                                             ctypes.c_int(z.shape[0]), ctypes.c_int(V), ctypes.c_int(ctx.start),
                                             ctypes.c_longlong(ctx.ignore_index), _lib.stream_ptr()), "axb_ce_bwd")
            return z.reshape(ctx.shape), None, None, None
        p = (z.float() - lse[:, None]).exp()
        loc = t - ctx.start
        inside = (loc >= 0) & (loc < V)
        onehot = torch.zeros_like(p)
        onehot[inside, loc[inside]] = 1.0
        valid = (t != ctx.ignore_index).float()[:, None]
        return ((p - onehot) * valid * scale).to(z.dtype).reshape(ctx.shape), None, None, None


def cross_entropy(logits, targets, group=None, ignore_index=-100):
    """Mean token cross-entropy.  With ``group`` the last dimension of ``logits``
    is this rank's contiguous slice of the vocabulary (rank order = slice order).
    On GPU the logits buffer is consumed: backward overwrites it with the gradient."""
    return _CrossEntropyFn.apply(logits, targets, group, ignore_index)
