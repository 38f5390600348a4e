"""Python entry points of the fused compute+collective kernels.

``gemm_all_reduce`` runs a tensor-parallel GEMM whose epilogue performs the
all-reduce over the group by exchanging partial output tiles through
peer-mapped ("symmetric") memory over NVLink, inside the GEMM kernel
(``csrc/gemm_tcgen05.cu``, ``AxbArCtx``).  It replaces the pair
``matmul`` + ``dist.all_reduce`` of the reference's
``axonn/intra_layer/fully_connected.py:118-119,140-145``.

The ``try_*`` helpers return ``None``/``False`` when the fused path does not
apply (CPU tensors, ``AXONN_BACKEND=nccl``, group of one, unsupported group
size); the caller then uses ``torch.distributed``.
"""

import ctypes

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops.gemm import _DT, EPI_NONE
from . import symm

_BM = 128
_CTRL_BYTES = 4096


class AxbArCtx(ctypes.Structure):
    _fields_ = [
        ("n", ctypes.c_int), ("rank", ctypes.c_int), ("epoch", ctypes.c_uint), ("bn", ctypes.c_int),
        ("inbox_local", ctypes.c_void_p), ("inbox_peer", ctypes.c_void_p * 8),
        ("flags_local", ctypes.c_void_p), ("flags_peer", ctypes.c_void_p * 8),
        ("done_local", ctypes.c_void_p), ("done_peer", ctypes.c_void_p * 8),
        ("counter", ctypes.c_void_p),
        ("inbox_vecs_per_src", ctypes.c_ulonglong), ("flags_per_src", ctypes.c_ulonglong),
        ("mode", ctypes.c_int), ("rows_per_shard", ctypes.c_int),
    ]


class _ArChannel:
    """Symmetric buffers and call counter of the fused all-reduce for one group.

    Layout of the symmetric allocation (same on every rank):
      [0, 4096)        control: done[n] (u32) at 0, CTA counter (u32) at 256
      flags[parity]    n * flags_per_src u32
      inbox[parity]    n * inbox_vecs_per_src 16-byte words
    """

    def __init__(self, group):
        self.group = group
        self.n = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.epoch = 1
        self.flags_per_src = 0
        self.inbox_vecs_per_src = 0
        self.buf = None

    def _layout(self):
        fbytes = self.n * self.flags_per_src * 4
        ibytes = self.n * self.inbox_vecs_per_src * 16
        f0 = _CTRL_BYTES
        i0 = (f0 + 2 * fbytes + 1023) // 1024 * 1024
        return f0, fbytes, i0, ibytes, i0 + 2 * ibytes

    def ensure(self, tiles, bn):
        need_flags = tiles * 4
        need_vecs = tiles * 4 * (bn // 32) * 128
        if need_flags <= self.flags_per_src and need_vecs <= self.inbox_vecs_per_src:
            return
        self.flags_per_src = max(self.flags_per_src, (need_flags + 1023) // 1024 * 1024)
        self.inbox_vecs_per_src = max(self.inbox_vecs_per_src, need_vecs)
        total = self._layout()[4]
        torch.cuda.synchronize()
        self.buf = symm.SymmBuffer(self.group, total, "gemm_ar")
        self.buf.local.zero_()
        torch.cuda.synchronize()
        self.buf.barrier()
        dist.barrier(group=self.group)
        self.epoch = 1

    def context(self, bn, mode=0, rows_per_shard=0):
        self.epoch += 1
        parity = self.epoch & 1
        f0, fbytes, i0, ibytes, _ = self._layout()
        c = AxbArCtx()
        c.n, c.rank, c.epoch, c.bn = self.n, self.rank, self.epoch, bn
        base = self.buf.peer_ptrs
        me = base[self.rank]
        c.inbox_local = me + i0 + parity * ibytes
        c.flags_local = me + f0 + parity * fbytes
        c.done_local = me
        c.counter = me + 256
        for j in range(self.n):
            c.inbox_peer[j] = base[j] + i0 + parity * ibytes
            c.flags_peer[j] = base[j] + f0 + parity * fbytes
            c.done_peer[j] = base[j]
        c.inbox_vecs_per_src = self.inbox_vecs_per_src
        c.flags_per_src = self.flags_per_src
        c.mode, c.rows_per_shard = mode, rows_per_shard
        return c


_channels = {}


def reset():
    _channels.clear()


def usable(group, tensor) -> bool:
    if not (tensor.is_cuda and symm.enabled()):
        return False
    n = dist.get_world_size(group)
    return 2 <= n <= 8


def gemm_all_reduce(layout, a, b, group, bias=None, epilogue=EPI_NONE, aux=None, out_dtype=None):
    """``all_reduce(op(a) @ op(b))`` over ``group`` (+bias, +GELU) in one kernel.

    layout 0: a[M,K] b[N,K] -> a b^T; layout 1: a[M,K] b[K,N] -> a b.  Every
    rank of the group must call this with the same shapes, in the same order."""
    M, K = a.shape
    N = b.shape[0] if layout == 0 else b.shape[1]
    a = a if a.is_contiguous() else a.contiguous()
    b = b if b.is_contiguous() else b.contiguous()
    ch = _channels.get(id(group))
    if ch is None:
        ch = _channels[id(group)] = _ArChannel(group)
    tiles_m = (M + _BM - 1) // _BM
    bn = 256 if tiles_m * ((N + 255) // 256) >= 148 else 128
    tiles = tiles_m * ((N + bn - 1) // bn)
    ch.ensure(tiles, bn)
    ctx = ch.context(bn)
    out = torch.empty((M, N), dtype=out_dtype or a.dtype, device=a.device)
    st = _lib.lib().axb_gemm_ar(
        ctypes.c_int(layout), _lib.ptr(a), _lib.ptr(b), _lib.ptr(out), _lib.ptr(bias), _lib.ptr(aux),
        ctypes.c_int(M), ctypes.c_int(N), ctypes.c_int(K), ctypes.c_int(_DT[a.dtype]), ctypes.c_int(_DT[out.dtype]),
        ctypes.c_int(epilogue), ctypes.c_int(a.device.index), _lib.stream_ptr(), ctypes.byref(ctx))
    _lib.check(st, "axb_gemm_ar")
    return out


def reduce_scatter_usable(group, tensor, rows) -> bool:
    n = dist.get_world_size(group)
    return usable(group, tensor) and rows % n == 0 and (rows // n) % 32 == 0


def gemm_reduce_scatter(layout, a, b, group, out_dtype=None, out=None, accumulate=False):
    """Row-wise ``reduce_scatter(op(a) @ op(b))`` over ``group`` in one kernel: rank ``o`` receives rows
    ``[o*R, (o+1)*R)`` of the summed product (``R = M / n``), optionally accumulated into ``out``.

    layout 2 (``a[K,M]``, ``b[K,N]`` -> ``a.T @ b``) is the weight-gradient product whose row blocks are
    exactly the depth shards of the flattened weight."""
    if layout == 2:
        K, M = a.shape
        N = b.shape[1]
    elif layout == 0:
        M, K = a.shape
        N = b.shape[0]
    else:
        M, K = a.shape
        N = b.shape[1]
    a = a if a.is_contiguous() else a.contiguous()
    b = b if b.is_contiguous() else b.contiguous()
    ch = _channels.get(id(group))
    if ch is None:
        ch = _channels[id(group)] = _ArChannel(group)
    R = M // ch.n
    tiles_m = (M + _BM - 1) // _BM
    bn = 256 if tiles_m * ((N + 255) // 256) >= 148 else 128
    tiles = tiles_m * ((N + bn - 1) // bn)
    ch.ensure(tiles, bn)
    ctx = ch.context(bn, mode=1, rows_per_shard=R)
    if out is None:
        out = torch.empty((R, N), dtype=out_dtype or a.dtype, device=a.device)
        accumulate = False
    st = _lib.lib().axb_gemm_rs(
        ctypes.c_int(layout), _lib.ptr(a), _lib.ptr(b), _lib.ptr(out), ctypes.c_int(M), ctypes.c_int(N),
        ctypes.c_int(K), ctypes.c_int(_DT[a.dtype]), ctypes.c_int(_DT[out.dtype]), ctypes.c_int(1 if accumulate else 0),
        ctypes.c_int(a.device.index), _lib.stream_ptr(), ctypes.byref(ctx))
    _lib.check(st, "axb_gemm_rs")
    return out


def try_all_reduce_scale_(grads, group, scale) -> bool:
    return False
