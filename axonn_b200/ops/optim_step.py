"""Fused multi-tensor AdamW step and top-k gradient pruning (``csrc/optim.cu``,
``csrc/prune.cu``)."""

import ctypes

import torch

from . import _lib
from .multi_tensor import _CHUNK, _DT_CODE


class AdamTable:
    """Device table for ``axb_multi_adamw``: one row per parameter."""

    def __init__(self, masters, models, grads, exp_avgs, exp_avg_sqs):
        rows, prefix = [], 0
        for p, mdl, g, m, v in zip(masters, models, grads, exp_avgs, exp_avg_sqs):
            assert p.dtype == torch.float32 and m.dtype == torch.float32 and v.dtype == torch.float32
            assert mdl is None or mdl.dtype == torch.bfloat16
            for t in (p, g, m, v):
                assert t.is_contiguous()
            rows.append((p.data_ptr(), 0 if mdl is None else mdl.data_ptr(), g.data_ptr(), m.data_ptr(),
                         v.data_ptr(), p.numel(), _DT_CODE[g.dtype], prefix))
            prefix += (p.numel() + _CHUNK - 1) // _CHUNK
        self.n, self.total_chunks = len(rows), prefix
        self.grad_ptrs = tuple(g.data_ptr() for g in grads)
        self.host = torch.tensor(rows, dtype=torch.int64).pin_memory()
        self.dev = self.host.to(masters[0].device, non_blocking=True)


def multi_tensor_adamw(table, lr, beta1, beta2, eps, weight_decay, step, grad_scale=None, found_inf=None):
    """One AdamW step for every tensor of ``table`` (an ``AdamTable``) in a single launch: fp32 master and
    moments updated, the 16-bit model copy written in the same pass; ``grad_scale`` (0-d device tensor) multiplies
    the gradients, a non-zero ``found_inf`` skips the update."""
    bc1 = 1.0 - beta1 ** step
    bc2 = 1.0 - beta2 ** step
    st = _lib.lib().axb_multi_adamw(
        _lib.ptr(table.dev), ctypes.c_int(table.n), ctypes.c_longlong(table.total_chunks), ctypes.c_float(lr),
        ctypes.c_float(beta1), ctypes.c_float(beta2), ctypes.c_float(eps), ctypes.c_float(weight_decay),
        ctypes.c_float(bc1), ctypes.c_float(bc2), _lib.ptr(grad_scale), _lib.ptr(found_inf), _lib.stream_ptr())
    _lib.check(st, "axb_multi_adamw")


def adamw_reference_(p, g, m, v, lr, beta1, beta2, eps, weight_decay, step, grad_scale=1.0):
    """Plain PyTorch AdamW update of one tensor (CPU path and test oracle)."""
    g = g.float() * grad_scale
    m.mul_(beta1).add_(g, alpha=1 - beta1)
    v.mul_(beta2).addcmul_(g, g, value=1 - beta2)
    bc1, bc2 = 1 - beta1 ** step, 1 - beta2 ** step
    denom = (v.sqrt() / (bc2 ** 0.5)).add_(eps)
    p.mul_(1 - lr * weight_decay).addcdiv_(m, denom, value=-lr / bc1)


_prune_ws = {}
# dtype codes of the C interface (csrc/axonn_b200.h)
_LIB_DTYPE = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}


def prune_topk_(grad, keep_fraction):
    """Zero all but the ``keep_fraction`` largest-magnitude entries of ``grad`` in place."""
    n = grad.numel()
    k = max(1, int(round(n * keep_fraction)))
    if k >= n:
        return grad
    if grad.is_cuda:
        assert grad.is_contiguous()
        L = _lib.lib()
        dev = grad.device
        ws = _prune_ws.get(dev)
        if ws is None:
            ws = torch.empty(L.axb_prune_workspace_words(), dtype=torch.int32, device=dev)
            _prune_ws[dev] = ws
        st = L.axb_prune_topk(_lib.ptr(grad), ctypes.c_longlong(n), ctypes.c_int(_LIB_DTYPE[grad.dtype]),
                              ctypes.c_longlong(k), _lib.ptr(ws), ctypes.c_int(dev.index), _lib.stream_ptr())
        _lib.check(st, "axb_prune_topk")
        _lib.add_launches(2)
        return grad
    flat = grad.view(-1)
    thr = flat.abs().float().kthvalue(n - k + 1).values
    flat.mul_((flat.abs().float() >= thr).to(flat.dtype))
    return grad
