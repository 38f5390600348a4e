"""Autograd-aware dense linear algebra on the package's GEMM kernels for layers
that are not tensor parallel (router, expert MLPs)."""

import torch

from .gemm import bmm_nn, bmm_nt, bmm_tn, matmul_nn, matmul_nt, matmul_tn


class _LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w):
        ctx.save_for_backward(x, w)
        x2 = x.reshape(-1, x.shape[-1])
        return matmul_nt(x2, w).reshape(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, g):
        x, w = ctx.saved_tensors
        g2 = g.reshape(-1, g.shape[-1])
        g2 = g2 if g2.is_contiguous() else g2.contiguous()
        x2 = x.reshape(-1, x.shape[-1])
        gx = matmul_nn(g2, w).reshape(x.shape) if ctx.needs_input_grad[0] else None
        gw = matmul_tn(g2, x2, out_dtype=w.dtype) if ctx.needs_input_grad[1] else None
        return gx, gw


def linear(x, w):
    """``x @ w.T`` for ``w`` of shape ``[out, in]``."""
    if x.shape[0] == 0 or x.numel() == 0:
        return x.new_zeros(*x.shape[:-1], w.shape[0]) + 0 * w.sum()
    return _LinearFn.apply(x, w)


class _BatchedLinearFn(torch.autograd.Function):
    """``y[e] = x[e] @ w[e].T`` for all ``e`` with one kernel launch per GEMM of forward and backward."""

    @staticmethod
    def forward(ctx, x, w, seg, seg_rows):
        ctx.save_for_backward(x, w)
        ctx.seg, ctx.seg_rows = seg, seg_rows
        return bmm_nt(x, w, seg=seg, seg_rows=seg_rows)

    @staticmethod
    def backward(ctx, g):
        x, w = ctx.saved_tensors
        g = g if g.is_contiguous() else g.contiguous()
        gx = bmm_nn(g, w, seg=ctx.seg, seg_rows=ctx.seg_rows) if ctx.needs_input_grad[0] else None
        gw = bmm_tn(g, x, out_dtype=w.dtype, seg=ctx.seg, seg_rows=ctx.seg_rows) if ctx.needs_input_grad[1] else None
        return gx, gw, None, None


def linear_batched(x, w, seg=None, seg_rows=0):
    """``x[E, rows, in] @ w[E, out, in].T`` -> ``[E, rows, out]``: the expert GEMMs of a mixture-of-experts layer
    as one launch over the tiles of all experts (instead of one launch per expert).

    ``seg`` (int32 ``[E, rows / seg_rows]``, on the device): the rows of every problem are segments of ``seg_rows``
    rows of which only the first ``seg[e, s]`` hold data and the rest are ZERO (capacity padding).  The kernels
    then skip the tiles without data - the output rows of skipped tiles are zeros, which is what the full product
    would give when the layer has no bias."""
    return _BatchedLinearFn.apply(x, w, seg, seg_rows)
