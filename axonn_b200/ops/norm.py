"""LayerNorm and RMSNorm (forward + backward kernels in ``csrc/norm.cu``).

Both accept a hidden dimension that is sharded over a process group
(``group``): the per-row statistics are then partial sums that are all-reduced
between a "statistics" launch and an "apply" launch, in forward and backward.
They stand in for the apex fused LayerNorm and the HF RMSNorm that the
reference's models rely on (``external/models/nvidia_transformer.py:57-95``,
``axonn/models/transformers/modify_llama.py``).
"""

import ctypes

import torch
import torch.distributed as dist

from . import _lib

_DT = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}


def _group_size(group):
    return 1 if group is None else dist.get_world_size(group)


def _torch_norm_fwd(x, gamma, beta, eps, rms, group):
    xf = x.float()
    n = _group_size(group)
    H_total = x.shape[-1] * n
    s2 = xf.pow(2).sum(-1, keepdim=True)
    s1 = torch.zeros_like(s2) if rms else xf.sum(-1, keepdim=True)
    if n > 1:
        st = torch.cat([s1, s2], -1)
        dist.all_reduce(st, group=group)
        s1, s2 = st[..., :1], st[..., 1:]
    mean = s1 / H_total
    var = s2 / H_total - (0 if rms else mean * mean)
    rstd = torch.rsqrt(var.clamp_min(0) + eps)
    y = (xf - mean) * rstd * gamma.float()
    if beta is not None:
        y = y + beta.float()
    return y.to(x.dtype), mean, rstd


class _NormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gamma, beta, eps, rms, group):
        shape = x.shape
        H = shape[-1]
        x2 = x.reshape(-1, H).contiguous()
        rows = x2.shape[0]
        n = _group_size(group)
        ctx.rms, ctx.group, ctx.n, ctx.shape, ctx.has_beta = rms, group, n, shape, beta is not None
        if not x2.is_cuda:
            y, mean, rstd = _torch_norm_fwd(x2, gamma, beta, eps, rms, group)
            ctx.save_for_backward(x2, gamma, mean, rstd)
            return y.reshape(shape)
        L = _lib.lib()
        dev = x2.device.index
        y = torch.empty_like(x2)
        stats = torch.empty((rows, 2), dtype=torch.float32, device=x2.device)
        g = gamma.to(x2.dtype) if gamma.dtype != x2.dtype else gamma
        b = None if beta is None else (beta.to(x2.dtype) if beta.dtype != x2.dtype else beta)

        def call(mode):
            st = L.axb_norm_fwd(_lib.ptr(x2), _lib.ptr(g), _lib.ptr(b), _lib.ptr(y), _lib.ptr(stats),
                                ctypes.c_int(rows), ctypes.c_int(H), ctypes.c_int(H * n), ctypes.c_float(eps),
                                ctypes.c_int(1 if rms else 0), ctypes.c_int(mode), ctypes.c_int(_DT[x2.dtype]),
                                ctypes.c_int(dev), _lib.stream_ptr())
            _lib.check(st, "axb_norm_fwd")

        if n == 1:
            call(0)
        else:
            call(1)                              # partial (sum x, sum x^2) of my slice of the hidden dimension
            dist.all_reduce(stats, group=group)
            call(3)                              # finishes (mean, rstd) in place and applies them
        ctx.save_for_backward(x2, g, stats)
        return y.reshape(shape)

    @staticmethod
    def backward(ctx, dy):
        rms, group, n = ctx.rms, ctx.group, ctx.n
        H = ctx.shape[-1]
        dy2 = dy.reshape(-1, H).contiguous()
        if not dy2.is_cuda:
            x2, gamma, mean, rstd = ctx.saved_tensors
            xh = (x2.float() - mean) * rstd
            gd = dy2.float() * gamma.float()
            s1 = torch.zeros_like(mean) if rms else gd.sum(-1, keepdim=True)
            s2 = (gd * xh).sum(-1, keepdim=True)
            if n > 1:
                st = torch.cat([s1, s2], -1)
                dist.all_reduce(st, group=group)
                s1, s2 = st[..., :1], st[..., 1:]
            Ht = H * n
            dx = rstd * (gd - s1 / Ht - xh * s2 / Ht)
            dgamma = (dy2.float() * xh).sum(0).to(gamma.dtype)
            dbeta = dy2.float().sum(0).to(gamma.dtype) if ctx.has_beta else None
            return dx.to(dy.dtype).reshape(ctx.shape), dgamma, dbeta, None, None, None
        x2, g, stats = ctx.saved_tensors
        rows = x2.shape[0]
        L = _lib.lib()
        dev = x2.device.index
        grid = L.axb_norm_grid(ctypes.c_int(dev), ctypes.c_int(rows))
        dx = torch.empty_like(x2)
        sums = torch.empty((rows, 2), dtype=torch.float32, device=x2.device) if n > 1 else None
        part = torch.empty((2, grid, H), dtype=torch.float32, device=x2.device)
        dgb = torch.empty((2, H), dtype=g.dtype, device=x2.device)   # written in the parameter's dtype: no cast kernel

        def call(mode):
            st = L.axb_norm_bwd(_lib.ptr(dy2), _lib.ptr(x2), _lib.ptr(g), _lib.ptr(stats), _lib.ptr(dx),
                                _lib.ptr(sums), _lib.ptr(part[0]), _lib.ptr(part[1]), _lib.ptr(dgb[0]),
                                _lib.ptr(dgb[1]), ctypes.c_int(rows), ctypes.c_int(H), ctypes.c_int(H * n),
                                ctypes.c_int(1 if rms else 0), ctypes.c_int(mode), ctypes.c_int(_DT[x2.dtype]),
                                ctypes.c_int(_DT[g.dtype]), ctypes.c_int(dev), _lib.stream_ptr())
            _lib.check(st, "axb_norm_bwd")
            if mode != 1:
                _lib.add_launches(1)

        if n == 1:
            call(0)
        else:
            call(1)
            dist.all_reduce(sums, group=group)
            call(2)
        dgamma = dgb[0]
        dbeta = dgb[1] if ctx.has_beta else None
        return dx.reshape(ctx.shape), dgamma, dbeta, None, None, None


class _AddNormFn(torch.autograd.Function):
    """``h = x + delta``; ``y = norm(h)``; returns ``(h, y)``.  On CUDA the add is done inside the norm kernel
    (one read of ``x`` and ``delta``, one write of ``h`` and ``y``) and the backward adds the gradient of the
    residual path to the norm's input gradient inside the backward kernel; elsewhere it is the two plain steps."""

    @staticmethod
    def forward(ctx, x, delta, gamma, beta, eps, rms, group):
        shape = x.shape
        H = shape[-1]
        n = _group_size(group)
        ctx.rms, ctx.group, ctx.n, ctx.shape, ctx.has_beta = rms, group, n, shape, beta is not None
        x2 = x.reshape(-1, H).contiguous()
        d2 = delta.reshape(-1, H).contiguous()
        rows = x2.shape[0]
        if not x2.is_cuda:
            h = x2 + d2
            y, mean, rstd = _torch_norm_fwd(h, gamma, beta, eps, rms, group)
            ctx.save_for_backward(h, gamma, mean, rstd)
            return h.reshape(shape), y.reshape(shape)
        L = _lib.lib()
        dev = x2.device.index
        h = torch.empty_like(x2)
        y = torch.empty_like(x2)
        stats = torch.empty((rows, 2), dtype=torch.float32, device=x2.device)
        g = gamma.to(x2.dtype) if gamma.dtype != x2.dtype else gamma
        b = None if beta is None else (beta.to(x2.dtype) if beta.dtype != x2.dtype else beta)

        def call(mode, src, dl):
            st = L.axb_add_norm_fwd(_lib.ptr(src), _lib.ptr(dl), _lib.ptr(h if dl is not None else None), _lib.ptr(g),
                                    _lib.ptr(b), _lib.ptr(y), _lib.ptr(stats), ctypes.c_int(rows), ctypes.c_int(H),
                                    ctypes.c_int(H * n), ctypes.c_float(eps), ctypes.c_int(1 if rms else 0),
                                    ctypes.c_int(mode), ctypes.c_int(_DT[x2.dtype]), ctypes.c_int(dev), _lib.stream_ptr())
            _lib.check(st, "axb_add_norm_fwd")

        if n == 1:
            call(0, x2, d2)
        else:
            call(1, x2, d2)                      # writes h and the partial row sums
            dist.all_reduce(stats, group=group)
            call(3, h, None)                     # finishes (mean, rstd) in place and applies them
        ctx.save_for_backward(h, g, stats)
        return h.reshape(shape), y.reshape(shape)

    @staticmethod
    def backward(ctx, dh, dy):
        rms, group, n = ctx.rms, ctx.group, ctx.n
        H = ctx.shape[-1]
        dy2 = dy.reshape(-1, H).contiguous()
        dh2 = None if dh is None else dh.reshape(-1, H).contiguous()
        if not dy2.is_cuda:
            x2, gamma, mean, rstd = ctx.saved_tensors
            xh = (x2.float() - mean) * rstd
            gd = dy2.float() * gamma.float()
            s1 = torch.zeros_like(mean) if rms else gd.sum(-1, keepdim=True)
            s2 = (gd * xh).sum(-1, keepdim=True)
            if n > 1:
                st = torch.cat([s1, s2], -1)
                dist.all_reduce(st, group=group)
                s1, s2 = st[..., :1], st[..., 1:]
            Ht = H * n
            dx = rstd * (gd - s1 / Ht - xh * s2 / Ht)
            if dh2 is not None:
                dx = dx + dh2.float()
            dgamma = (dy2.float() * xh).sum(0).to(gamma.dtype)
            dbeta = dy2.float().sum(0).to(gamma.dtype) if ctx.has_beta else None
            dx = dx.to(dy.dtype).reshape(ctx.shape)
            return dx, dx, dgamma, dbeta, None, None, None
        x2, g, stats = ctx.saved_tensors
        rows = x2.shape[0]
        L = _lib.lib()
        dev = x2.device.index
        grid = L.axb_norm_grid(ctypes.c_int(dev), ctypes.c_int(rows))
        dx = torch.empty_like(x2)
        sums = torch.empty((rows, 2), dtype=torch.float32, device=x2.device) if n > 1 else None
        part = torch.empty((2, grid, H), dtype=torch.float32, device=x2.device)
        dgb = torch.empty((2, H), dtype=g.dtype, device=x2.device)

        def call(mode):
            st = L.axb_add_norm_bwd(_lib.ptr(dy2), _lib.ptr(dh2), _lib.ptr(x2), _lib.ptr(g), _lib.ptr(stats), _lib.ptr(dx),
                                    _lib.ptr(sums), _lib.ptr(part[0]), _lib.ptr(part[1]), _lib.ptr(dgb[0]),
                                    _lib.ptr(dgb[1]), ctypes.c_int(rows), ctypes.c_int(H), ctypes.c_int(H * n),
                                    ctypes.c_int(1 if rms else 0), ctypes.c_int(mode), ctypes.c_int(_DT[x2.dtype]),
                                    ctypes.c_int(_DT[g.dtype]), ctypes.c_int(dev), _lib.stream_ptr())
            _lib.check(st, "axb_add_norm_bwd")
            if mode != 1:
                _lib.add_launches(1)

        if n == 1:
            call(0)
        else:
            call(1)
            dist.all_reduce(sums, group=group)
            call(2)
        dx = dx.reshape(ctx.shape)
        return dx, dx, dgb[0], (dgb[1] if ctx.has_beta else None), None, None, None


def add_layer_norm(x, delta, gamma, beta, eps=1e-5, group=None):
    """``h = x + delta; y = LayerNorm(h)`` in one kernel; returns ``(h, y)``."""
    return _AddNormFn.apply(x, delta, gamma, beta, eps, False, group)


def add_rms_norm(x, delta, gamma, eps=1e-6, group=None):
    """``h = x + delta; y = RMSNorm(h)`` in one kernel; returns ``(h, y)``."""
    return _AddNormFn.apply(x, delta, gamma, None, eps, True, group)


def layer_norm(x, gamma, beta, eps=1e-5, group=None):
    """LayerNorm over the last dimension; with ``group`` the last dimension is one
    shard of a hidden dimension split over that process group."""
    return _NormFn.apply(x, gamma, beta, eps, False, group)


def rms_norm(x, gamma, eps=1e-6, group=None):
    """RMSNorm over the last dimension; with ``group`` the last dimension is one shard of a hidden dimension
    split over that process group."""
    return _NormFn.apply(x, gamma, None, eps, True, group)


def column_sum(x, out_dtype=torch.float32):
    """``x.sum(0)`` of a 2-D tensor, accumulated in fp32 and returned as ``out_dtype`` (bias gradients).  One
    pass over ``x`` at memory bandwidth on CUDA (partial sums per row split, then a fold that writes the
    requested dtype); plain PyTorch elsewhere."""
    if not (_lib.use_cuda_kernels(x) and x.dim() == 2 and x.shape[1] % 8 == 0 and x.is_contiguous()
            and x.dtype in (torch.bfloat16, torch.float16, torch.float32) and x.shape[0] > 0
            and out_dtype in _DT):
        return x.sum(0, dtype=torch.float32).to(out_dtype)
    rows, n = x.shape
    L = _lib.lib()
    dev = x.device.index
    splits = L.axb_colsum_splits(ctypes.c_int(dev), ctypes.c_int(rows), ctypes.c_int(n))
    part = torch.empty((splits, n), dtype=torch.float32, device=x.device)
    out = torch.empty(n, dtype=out_dtype, device=x.device)
    _lib.check(L.axb_colsum(_lib.ptr(x), _lib.ptr(part), _lib.ptr(out), ctypes.c_int(rows), ctypes.c_int(n),
                            ctypes.c_int(_DT[x.dtype]), ctypes.c_int(_DT[out_dtype]), ctypes.c_int(dev),
                            _lib.stream_ptr()), "axb_colsum")
    _lib.add_launches(1)
    return out
