"""Autograd-aware dense linear algebra on the package's GEMM kernels for layers
that are not tensor parallel (router, expert MLPs)."""

import torch

from .gemm import matmul_nn, matmul_nt, matmul_tn


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
