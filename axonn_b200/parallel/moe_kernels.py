"""Peer-memory MoE token exchange: autograd wrappers and flag protocol for the
dispatch / combine kernels of ``csrc/moe.cu``.

Each expert-parallel group owns one symmetric allocation per rank:

    control block   FILLED_X[n] FREE_X[n] READY_Y[n] PULLED_Y[n] (u32 epochs), CTA counter,
                    COUNTS[local expert][source] (rows of each capacity segment that hold tokens)
    X buffer        [local expert][source][capacity][hidden]   tokens arriving for my experts
    Y buffer        same shape                                  my experts' outputs, pulled by the sources

The expert-major layout makes the X buffer the stacked operand of the batched expert GEMM as it is, and
COUNTS lets that GEMM skip the tiles of the capacity padding (``axb_gemm_batched``'s row mask).

``scatter`` stores rows into the owners' X buffers (FREE_X gates the stores,
FILLED_X tells the owner they are complete); ``gather`` pulls rows from the
owners' Y buffers (READY_Y gates the loads, PULLED_Y lets the owner reuse Y).
The two are each other's adjoint, so forward dispatch/combine and their
backward passes are the same two kernels.
"""

import ctypes

import torch
import torch.distributed as dist

from ..ops import _lib
from . import symm

_FILLED_X, _FREE_X, _READY_Y, _PULLED_Y, _COUNTER, _COUNTS = 0, 64, 128, 192, 1024, 2048
_CTRL = 4096


class AxbMoeCtx(ctypes.Structure):
    _fields_ = [("n", ctypes.c_int), ("rank", ctypes.c_int), ("epoch", ctypes.c_uint), ("n_local", ctypes.c_int),
                ("buf_peer", ctypes.c_void_p * 8), ("wait_local", ctypes.c_void_p), ("wait_value", ctypes.c_uint),
                ("signal_peer", ctypes.c_void_p * 8), ("counter", ctypes.c_void_p), ("cnt_peer", ctypes.c_void_p * 8)]


DISABLED = False     # benchmarks flip this to time the all_to_all_single path on the same layer


def usable(group, x) -> bool:
    if DISABLED or not (x.is_cuda and symm.enabled() and x.dtype == torch.bfloat16):
        return False
    n = dist.get_world_size(group)
    if n < 2 or n > 8:
        return False
    return hasattr(_lib.lib(), "axb_moe_dispatch")


class _Channel:
    def __init__(self, group, n_local, C, H):
        self.group, self.n, self.rank = group, dist.get_world_size(group), dist.get_rank(group)
        self.n_local, self.C, self.H = n_local, C, H
        self.buf_bytes = self.n * n_local * C * H * 2
        self.x_off = _CTRL
        self.y_off = _CTRL + (self.buf_bytes + 1023) // 1024 * 1024
        total = self.y_off + self.buf_bytes
        torch.cuda.synchronize()
        self.buf = symm.SymmBuffer(group, total, "moe")
        self.buf.local.zero_()
        torch.cuda.synchronize()
        self.buf.barrier()
        dist.barrier(group=group)
        self.epoch_x = 0
        self.epoch_y = 0
        self.device = self.buf.local.device

    def view(self, off):
        return self.buf.local[off:off + self.buf_bytes].view(torch.bfloat16).view(
            self.n_local, self.n, self.C, self.H)

    def counts_view(self):
        return self.buf.local[_COUNTS:_COUNTS + self.n_local * self.n * 4].view(torch.int32).view(self.n_local, self.n)

    def ctx(self, epoch, buf_off, wait_off, wait_value, signal_off):
        c = AxbMoeCtx()
        c.n, c.rank, c.epoch, c.n_local = self.n, self.rank, epoch, self.n_local
        base = self.buf.peer_ptrs
        for j in range(self.n):
            c.buf_peer[j] = base[j] + buf_off
            c.signal_peer[j] = base[j] + signal_off
        c.wait_local = base[self.rank] + wait_off
        c.wait_value = max(0, wait_value)
        c.counter = base[self.rank] + _COUNTER
        return c

    # -- primitives -----------------------------------------------------------------
    def scatter(self, rows, by_token, dest, keep, counts, T, k):
        """rows -> owners' X buffers; returns my experts' inputs [n_local, n*C, H] (a copy) and the int32 table
        [n_local, n] of how many rows of each source's capacity segment hold tokens."""
        L = _lib.lib()
        dev = self.device.index
        self.epoch_x += 1
        e = self.epoch_x
        c = self.ctx(e, self.x_off, _FREE_X, e - 1, _FILLED_X)
        for j in range(self.n):
            c.cnt_peer[j] = self.buf.peer_ptrs[j] + _COUNTS
        _lib.check(L.axb_moe_dispatch(_lib.ptr(rows), ctypes.c_int(1 if by_token else 0), _lib.ptr(dest),
                                      _lib.ptr(keep), _lib.ptr(counts), ctypes.c_int(T), ctypes.c_int(k),
                                      ctypes.c_int(self.n * self.n_local), ctypes.c_int(self.C),
                                      ctypes.c_int(self.H), ctypes.byref(c), ctypes.c_int(dev), _lib.stream_ptr()),
                   "axb_moe_dispatch")
        w = self.ctx(e, self.x_off, _FILLED_X, e, _FREE_X)
        _lib.check(L.axb_moe_wait(ctypes.byref(w), ctypes.c_int(dev), _lib.stream_ptr()), "axb_moe_wait")
        mine = self.view(self.x_off).reshape(self.n_local, self.n * self.C, self.H).clone()
        seg = self.counts_view().clone()
        _lib.check(L.axb_moe_signal(ctypes.byref(w), ctypes.c_int(dev), _lib.stream_ptr()), "axb_moe_signal")
        return mine, seg

    def gather(self, y_local, dest, keep, T, k):
        """my experts' outputs [n_local, n*C, H] -> Y buffer; returns the rows of my assignments [T*k, H]."""
        L = _lib.lib()
        dev = self.device.index
        self.epoch_y += 1
        e = self.epoch_y
        w = self.ctx(e, self.y_off, _PULLED_Y, e - 1, _READY_Y)
        _lib.check(L.axb_moe_wait(ctypes.byref(w), ctypes.c_int(dev), _lib.stream_ptr()), "axb_moe_wait")
        self.view(self.y_off).copy_(y_local.reshape(self.n_local, self.n, self.C, self.H))
        _lib.check(L.axb_moe_signal(ctypes.byref(w), ctypes.c_int(dev), _lib.stream_ptr()), "axb_moe_signal")
        out = torch.empty((T * k, self.H), dtype=torch.bfloat16, device=self.device)
        c = self.ctx(e, self.y_off, _READY_Y, e, _PULLED_Y)
        _lib.check(L.axb_moe_gather(_lib.ptr(out), _lib.ptr(dest), _lib.ptr(keep), ctypes.c_int(T), ctypes.c_int(k),
                                    ctypes.c_int(self.C), ctypes.c_int(self.H), ctypes.byref(c), ctypes.c_int(dev),
                                    _lib.stream_ptr()), "axb_moe_gather")
        return out


_channels = {}


def reset():
    _channels.clear()


def _channel(group, n_local, C, H):
    key = (id(group), n_local, C, H)
    ch = _channels.get(key)
    if ch is None:
        ch = _channels[key] = _Channel(group, n_local, C, H)
    return ch


class _Scatter(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x2, dest, keep, counts, ch, k):
        ctx.ch, ctx.k, ctx.T = ch, k, x2.shape[0]
        ctx.save_for_backward(dest, keep)
        xin, seg = ch.scatter(x2.contiguous(), True, dest, keep, counts, x2.shape[0], k)
        ctx.mark_non_differentiable(seg)
        return xin, seg

    @staticmethod
    def backward(ctx, g, _seg_grad=None):
        dest, keep = ctx.saved_tensors
        picked = ctx.ch.gather(g.contiguous(), dest, keep, ctx.T, ctx.k)
        return picked.view(ctx.T, ctx.k, -1).sum(1), None, None, None, None, None


class _Gather(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y_local, dest, keep, counts, ch, T, k):
        ctx.ch, ctx.k, ctx.T = ch, k, T
        ctx.save_for_backward(dest, keep, counts)
        return ch.gather(y_local.contiguous(), dest, keep, T, k)

    @staticmethod
    def backward(ctx, g):
        dest, keep, counts = ctx.saved_tensors
        gy, _ = ctx.ch.scatter(g.contiguous(), False, dest, keep, counts, ctx.T, ctx.k)
        return gy, None, None, None, None, None, None


def dispatch_experts_combine(layer, x2, dest, keep, gate, capacity):
    """Route ``x2`` [T, H] through ``layer``'s experts over peer memory."""
    T, H = x2.shape
    k, E = layer.top_k, layer.n_experts
    ch = _channel(layer.group, layer.n_local, capacity, H)
    dest = dest.contiguous()
    keep_u8 = keep.to(torch.uint8).contiguous()
    counts = torch.zeros(E, dtype=torch.int64, device=x2.device)
    counts.index_add_(0, torch.div(dest, capacity, rounding_mode="floor"), keep.to(torch.int64))
    xin, seg = _Scatter.apply(x2, dest, keep_u8, counts, ch, k)
    out = layer._experts(xin, seg, capacity)
    picked = _Gather.apply(out, dest, keep_u8, counts, ch, T, k)
    w = (gate * keep).to(picked.dtype)
    return (picked.view(T, k, H) * w.view(T, k, 1)).sum(1)
