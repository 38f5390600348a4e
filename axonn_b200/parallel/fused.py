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


def _tile_geometry(M, N):
    """(tile width, number of tile indices) the kernel uses for an M x N product: 256-wide tiles when they
    fill the GPU, and tile rows rounded up to an even count because CTA pairs index tiles by (pair, CTA)."""
    tiles_m = (M + _BM - 1) // _BM
    bn = 256 if tiles_m * ((N + 255) // 256) >= 148 else 128
    return bn, (tiles_m + 1) // 2 * 2 * ((N + bn - 1) // bn)


class AxbArCtx(ctypes.Structure):
    _fields_ = [
        ("n", ctypes.c_int), ("rank", ctypes.c_int), ("epoch", ctypes.c_uint), ("bn", ctypes.c_int),
        ("inbox_local", ctypes.c_void_p), ("inbox_peer", ctypes.c_void_p * 8),
        ("flags_local", ctypes.c_void_p), ("flags_peer", ctypes.c_void_p * 8),
        ("done_local", ctypes.c_void_p), ("done_peer", ctypes.c_void_p * 8),
        ("counter", ctypes.c_void_p),
        ("inbox_vecs_per_src", ctypes.c_ulonglong), ("flags_per_src", ctypes.c_ulonglong),
        ("mode", ctypes.c_int), ("rows_per_shard", ctypes.c_int),
        ("comm_ctas", ctypes.c_int), ("loopback", ctypes.c_int),
        ("c_off", ctypes.c_ulonglong), ("aux_off", ctypes.c_ulonglong),
        ("arena_peer", ctypes.c_void_p * 8),
        ("mail_local", ctypes.c_void_p), ("mail_peer", ctypes.c_void_p * 8),
    ]


MODE_ONE_SHOT, MODE_REDUCE_SCATTER, MODE_TWO_SHOT = 0, 1, 2
_MAIL_OFF = 512   # mailbox of the two-shot all-reduce inside the control block: n records of 32 bytes


class _ArChannel:
    """Symmetric buffers and call counter of the fused all-reduce for one group.

    Layout of the symmetric allocation (same on every rank):
      [0, 4096)        control: done[n] (u32) at 0, CTA counter (u32) at 256, mailbox (n records of 8 u32:
                       offsets of a peer's C and aux in its output arena + epoch) at 512
      flags[parity]    n * flags_per_src u32   (indexed [source rank][tile * 4 + warp])
      inbox[parity]    n * inbox_vecs_per_src 16-byte words, indexed [source rank][tile][warp]: bf16 partial
                       tiles pushed by every rank's GEMM epilogue (the own ones stored locally)
    """

    def __init__(self, group):
        self.group = group
        self.n = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.epoch = 1
        self.flags_per_src = 0
        self.inbox_vecs_per_src = 0
        self.buf = None
        self.arena_bases = None

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
        c.comm_ctas = 0
        c.loopback = 0
        c.mail_local = me + _MAIL_OFF
        for j in range(self.n):
            c.mail_peer[j] = base[j] + _MAIL_OFF
        return c


_channels = {}


def reset():
    _channels.clear()
    _grad_channels.clear()
    _ag_channels.clear()
    _group_ok.clear()
    _a2a_channels.clear()
    _emb_channels.clear()
    _grad_ar_channels.clear()


_group_ok = {}


def _peer_capable(group) -> bool:
    """True when every rank of ``group`` sits on the same host, can address every other rank's GPU and a
    small symmetric allocation works.  Decided once per group, collectively (all ranks of the group reach
    their first fused call at the same layer), and the decision is agreed on with a MIN all-reduce so that no
    rank takes the fused path alone.  A group that spans hosts or lacks peer access keeps using
    ``torch.distributed``."""
    key = id(group)
    ok = _group_ok.get(key)
    if ok is not None:
        return ok
    import socket

    n = dist.get_world_size(group)
    ok, reason = True, ""
    try:
        me = (socket.gethostname(), torch.cuda.current_device())
        everyone = [None] * n
        dist.all_gather_object(everyone, me, group=group)
        if len({h for h, _ in everyone}) != 1:
            ok, reason = False, "the group's ranks are on different hosts"
        else:
            devs = [d for _, d in everyone]
            if len(set(devs)) != n:
                ok, reason = False, "several ranks of the group share one GPU"
            else:
                for d in devs:
                    if d != me[1] and not torch.cuda.can_device_access_peer(me[1], d):
                        ok, reason = False, f"GPU {me[1]} cannot address GPU {d}"
    except Exception as e:  # noqa: BLE001
        ok, reason = False, f"peer discovery failed: {e}"
    flag = torch.tensor([1 if ok else 0], dtype=torch.int32, device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
    ok = bool(flag.item())
    if ok:
        try:
            symm.SymmBuffer(group, 1 << 16, "probe")
        except Exception as e:  # noqa: BLE001
            ok, reason = False, f"symmetric allocation failed: {e}"
        flag.fill_(1 if ok else 0)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
        ok = bool(flag.item())
    if not ok:
        symm.disable(reason or "a peer rank could not use symmetric memory")
    _group_ok[key] = ok
    return ok


def group_usable(group, tensor) -> bool:
    """The peer-memory kernels can serve ``group`` for tensors on ``tensor``'s device."""
    if not (tensor.is_cuda and symm.enabled()):
        return False
    n = dist.get_world_size(group)
    return 2 <= n <= 8 and _peer_capable(group)


def usable(group, tensor, N=None, K=None, M=None) -> bool:
    """The fused GEMM kernels apply: peer-capable group, bf16/fp16 operands and, when given, dimensions
    that the tensor-core kernel accepts (N and K multiples of 8; M too for the transposed-A layout).
    Anything else (fp32 layers, odd widths) takes the ``matmul`` + ``torch.distributed`` path."""
    if tensor.dtype not in (torch.bfloat16, torch.float16):
        return False
    for d in (N, K, M):
        if d is not None and d % 8:
            return False
    return group_usable(group, tensor)


def _ar_outputs(ch, ctx, shape, dtype, device, want_aux):
    """Allocate C (and aux) of a fused all-reduce and complete ``ctx``: from the peer-mapped output arena
    with the two-shot protocol when the arena exists and the output is 16-bit, from ordinary memory with the
    one-shot protocol otherwise."""
    arena = symm.output_arena()
    if arena is not None and dtype in (torch.bfloat16, torch.float16):
        out = arena.empty(shape, dtype)
        aux = arena.empty(shape, dtype) if want_aux else None
        ctx.mode = MODE_TWO_SHOT
        ctx.c_off = arena.offset(out)
        ctx.aux_off = arena.offset(aux) if aux is not None else 0
        if ch.arena_bases is None:
            ch.arena_bases = arena.peer_bases(ch.group)
        for j, ptr in enumerate(ch.arena_bases):
            ctx.arena_peer[j] = ptr
    else:
        out = torch.empty(shape, dtype=dtype, device=device)
        aux = torch.empty(shape, dtype=dtype, device=device) if want_aux else None
    return out, aux


def gemm_all_reduce(layout, a, b, group, bias=None, epilogue=EPI_NONE, want_aux=False, out_dtype=None):
    """``all_reduce(op(a) @ op(b))`` over ``group`` (+bias, +GELU) in one kernel.

    layout 0: a[M,K] b[N,K] -> a b^T; layout 1: a[M,K] b[K,N] -> a b.  Every
    rank of the group must call this with the same shapes, in the same order.
    Returns the product, or ``(product, pre_activation)`` with ``want_aux`` (GELU epilogues).

    With a peer-mapped output arena (``symm.output_arena()``) the all-reduce is two-shot: every 32-row unit of
    a tile has one owner that receives the partials, sums them and stores the finished rows on every rank.
    For two ranks that is the NVLink volume of the one-shot form with half the stores, half the reduction
    work and 40 % less DRAM traffic per rank; for n ranks each element crosses NVLink 2 (n-1)/n times per rank
    instead of n-1.  Without the arena every rank receives and sums every partial (one-shot)."""
    M, K = a.shape
    N = b.shape[0] if layout == 0 else b.shape[1]
    a = a if a.is_contiguous() else a.contiguous()
    b = b if b.is_contiguous() else b.contiguous()
    ch = _channels.get(id(group))
    if ch is None:
        ch = _channels[id(group)] = _ArChannel(group)
    bn, tiles = _tile_geometry(M, N)
    ch.ensure(tiles, bn)
    ctx = ch.context(bn)
    out, aux = _ar_outputs(ch, ctx, (M, N), out_dtype or a.dtype, a.device, want_aux)
    st = _lib.lib().axb_gemm_ar(
        ctypes.c_int(layout), _lib.ptr(a), _lib.ptr(b), _lib.ptr(out), _lib.ptr(bias), _lib.ptr(aux),
        ctypes.c_int(M), ctypes.c_int(N), ctypes.c_int(K), ctypes.c_int(_DT[a.dtype]), ctypes.c_int(_DT[out.dtype]),
        ctypes.c_int(epilogue), ctypes.c_int(a.device.index), _lib.stream_ptr(), ctypes.byref(ctx))
    _lib.check(st, "axb_gemm_ar")
    return (out, aux) if want_aux else out


_loopback = {}


def gemm_all_reduce_loopback(a, b, bias=None, epilogue=EPI_NONE, out_dtype=None, silent_peer=False, two_shot=False):
    """Single-GPU emulation of a two-rank ``gemm_all_reduce`` (layout 0): the "peer" inbox, flags and done
    words are aliased onto this GPU's own slots of source rank 1, so one launch pushes its partial twice,
    reduces both copies and returns ``2 * (a @ b.T)`` (+bias, +GELU).  The kernel only ever waits on flags
    that its own CTAs raise.  It exercises the whole communication path of the kernel - epilogue pushes,
    flag publication, reducer warps, end-of-call handshake - with NVLink replaced by local stores, which is
    what a one-GPU test or a profiler capture of that path needs.

    ``silent_peer=True`` emulates a peer that never delivers: the flags of source rank 1 are redirected to a
    scratch area that nothing reads, so the kernel's wait for them runs into its deadline, the kernel returns
    and the status word reports it (``ops._lib.check_status``); the context stays usable.

    ``two_shot=True`` runs the two-shot protocol as rank 0 of 2: the units this rank owns (32-row groups with
    an even index) are stored for both source slots, reduced and written to the result and to a second buffer
    that stands in for the peer's ``C``; units owned by the "peer" are only pushed.  Returns ``(out, peer_out)``:
    both hold ``2 * (a @ b.T)`` in the owned rows, the other rows are never written."""
    M, K = a.shape
    N = b.shape[0]
    dev = a.device
    bn, tiles = _tile_geometry(M, N)
    flags_per_src = (tiles * 4 + 1023) // 1024 * 1024
    vecs_per_src = tiles * 4 * (bn // 32) * 128
    fbytes, ibytes = 2 * flags_per_src * 4, 2 * vecs_per_src * 16
    f0 = _CTRL_BYTES
    i0 = (f0 + 2 * fbytes + 1023) // 1024 * 1024
    total = i0 + 2 * ibytes
    st = _loopback.get(dev)
    if st is None or st["buf"].numel() < total or st["key"] != (flags_per_src, vecs_per_src):
        st = _loopback[dev] = {"buf": torch.zeros(total, dtype=torch.uint8, device=dev), "epoch": 1,
                               "key": (flags_per_src, vecs_per_src)}
    st["epoch"] += 1
    parity = st["epoch"] & 1
    me = st["buf"].data_ptr()
    c = AxbArCtx()
    c.n, c.rank, c.epoch, c.bn = 2, 0, st["epoch"], bn
    c.inbox_local = me + i0 + parity * ibytes
    c.flags_local = me + f0 + parity * fbytes
    c.done_local = me
    c.counter = me + 256
    c.inbox_peer[0], c.flags_peer[0], c.done_peer[0] = c.inbox_local, c.flags_local, me
    c.inbox_peer[1] = c.inbox_local + vecs_per_src * 16   # peer's slot of source 0 == own slot of source 1
    c.flags_peer[1] = c.flags_local + flags_per_src * 4
    if silent_peer:
        scratch = st.get("scratch")
        if scratch is None or scratch.numel() < flags_per_src * 4 * 2:
            scratch = st["scratch"] = torch.zeros(flags_per_src * 4 * 2, dtype=torch.uint8, device=dev)
        c.flags_peer[1] = scratch.data_ptr()   # flags[rank 0] of the "peer" land here: never seen locally
    c.done_peer[1] = me + 4                                # peer's done[0] == own done[1]
    c.inbox_vecs_per_src, c.flags_per_src = vecs_per_src, flags_per_src
    c.mode, c.rows_per_shard, c.comm_ctas = 0, 0, 0
    out = torch.empty((M, N), dtype=out_dtype or a.dtype, device=dev)
    peer_out = None
    if two_shot:
        peer_out = torch.empty_like(out)
        c.mode, c.loopback = MODE_TWO_SHOT, 1
        c.c_off, c.aux_off = 0, 0
        c.arena_peer[0], c.arena_peer[1] = out.data_ptr(), peer_out.data_ptr()
        c.mail_local = me + _MAIL_OFF
        c.mail_peer[0] = me + _MAIL_OFF
        c.mail_peer[1] = me + _MAIL_OFF + 32     # the "peer's" record of source 0 == own record of source 1
    rc = _lib.lib().axb_gemm_ar(
        ctypes.c_int(0), _lib.ptr(a), _lib.ptr(b), _lib.ptr(out), _lib.ptr(bias), _lib.ptr(None),
        ctypes.c_int(M), ctypes.c_int(N), ctypes.c_int(K), ctypes.c_int(_DT[a.dtype]), ctypes.c_int(_DT[out.dtype]),
        ctypes.c_int(epilogue), ctypes.c_int(dev.index), _lib.stream_ptr(), ctypes.byref(c))
    _lib.check(rc, "axb_gemm_ar")
    return (out, peer_out) if two_shot else out


def reduce_scatter_usable(group, a, b, rows) -> bool:
    """``a [K, rows]`` and ``b [K, N]`` of the transposed-A product whose row blocks are scattered."""
    n = dist.get_world_size(group)
    return (a.dtype == b.dtype and rows % n == 0 and (rows // n) % 32 == 0
            and usable(group, a, N=b.shape[1], K=a.shape[0], M=rows))


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
    bn, tiles = _tile_geometry(M, N)
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


class AxbAgCtx(ctypes.Structure):
    _fields_ = [("n", ctypes.c_int), ("rank", ctypes.c_int), ("epoch", ctypes.c_uint), ("n_copy", ctypes.c_int),
                ("outbox_peer", ctypes.c_void_p * 8), ("staging", ctypes.c_void_p),
                ("shard_bytes", ctypes.c_ulonglong), ("shard_ready", ctypes.c_void_p),
                ("ready_target", ctypes.c_uint), ("rows_per_shard", ctypes.c_int),
                ("wait_local", ctypes.c_void_p), ("done_peer", ctypes.c_void_p * 8), ("counter", ctypes.c_void_p)]


class _AgChannel:
    """Outboxes and flags of the fused all-gather -> GEMM for one (depth) group.
    Control block: READY[n] at 0, DONE[n] at 64, CTA counter at 256, shard arrival counters at 320;
    two outboxes (call parity) follow at 4096."""

    _READY, _DONE, _COUNTER, _SHARD_READY = 0, 64, 256, 320

    def __init__(self, group, shard_bytes):
        from .moe_kernels import AxbMoeCtx  # same flag-kernel context layout

        self._flag_ctx = AxbMoeCtx
        self.group, self.n, self.rank = group, dist.get_world_size(group), dist.get_rank(group)
        self.capacity = (int(shard_bytes) + (1 << 20) - 1) // (1 << 20) * (1 << 20)
        torch.cuda.synchronize()
        self.buf = symm.SymmBuffer(group, _CTRL_BYTES + 2 * self.capacity, "ag_gemm")
        self.buf.local.zero_()
        torch.cuda.synchronize()
        self.buf.barrier()
        dist.barrier(group=group)
        self.epoch = 1

    def publish(self, shard):
        """Copy my shard into this call's outbox and raise READY on every peer."""
        L = _lib.lib()
        self.epoch += 1
        e, parity = self.epoch, self.epoch & 1
        base = self.buf.peer_ptrs
        dev = shard.device.index
        c = self._flag_ctx()
        c.n, c.rank, c.epoch, c.n_local = self.n, self.rank, e, 1
        c.wait_local = base[self.rank] + self._DONE
        c.wait_value = max(0, e - 2)
        c.counter = base[self.rank] + self._COUNTER
        for j in range(self.n):
            c.buf_peer[j] = base[j]
            c.signal_peer[j] = base[j] + self._READY
        # one launch: wait until the peers are done with this parity's outbox (they read it in call e-2), copy the
        # shard into it, raise READY on every peer
        nbytes = shard.numel() * shard.element_size()
        off = _CTRL_BYTES + parity * self.capacity
        shard = shard.contiguous()
        _lib.check(L.axb_copy_publish(_lib.ptr(shard), ctypes.c_void_p(base[self.rank] + off), ctypes.c_longlong(nbytes),
                                      ctypes.byref(c), ctypes.c_int(dev), _lib.stream_ptr()), "axb_copy_publish")
        return e, parity, nbytes

    def context(self, e, parity, nbytes, staging, rows_per_shard, n_copy):
        base = self.buf.peer_ptrs
        c = AxbAgCtx()
        c.n, c.rank, c.epoch, c.n_copy = self.n, self.rank, e, n_copy
        for j in range(self.n):
            c.outbox_peer[j] = base[j] + _CTRL_BYTES + parity * self.capacity
            c.done_peer[j] = base[j] + self._DONE
        c.staging = staging.data_ptr()
        c.shard_bytes = nbytes
        c.shard_ready = base[self.rank] + self._SHARD_READY
        c.ready_target = n_copy
        c.rows_per_shard = rows_per_shard
        c.wait_local = base[self.rank] + self._READY
        c.counter = base[self.rank] + self._COUNTER
        return c


_ag_channels = {}


def all_gather_usable(group, x, w_shard, local_shape, layout) -> bool:
    if w_shard.dtype != x.dtype or not usable(group, x, N=local_shape[0], K=local_shape[1]):
        return False
    n = dist.get_world_size(group)
    rows = local_shape[0]
    if rows % n:
        return False
    R = rows // n
    if (w_shard.numel() * w_shard.element_size()) % 16:
        return False
    return R % 128 == 0 if layout == 0 else R % 64 == 0


def all_gather_gemm(layout, a, w_shard, depth_group, local_shape, ar_group=None, bias=None, epilogue=EPI_NONE,
                    want_aux=False):
    """``op(a) @ op(W)`` where ``W [out_l, in_l]`` is the row-wise concatenation of the depth group's flat
    shards: the gather runs inside the GEMM kernel.  layout 0: ``a[M,in_l] @ W.T``; layout 1:
    ``a[M,out_l] @ W``.  With ``ar_group`` the product is additionally all-reduced in the epilogue.
    Returns ``(product, W)`` — ``W`` is the gathered weight left behind by the kernel — or
    ``(product, W, pre_activation)`` with ``want_aux`` (GELU epilogues)."""
    out_l, in_l = local_shape
    M = a.shape[0]
    N, K = (out_l, in_l) if layout == 0 else (in_l, out_l)
    a = a if a.is_contiguous() else a.contiguous()
    ch = _ag_channels.get(id(depth_group))
    nbytes = w_shard.numel() * w_shard.element_size()
    if ch is None or ch.capacity < nbytes:
        ch = _ag_channels[id(depth_group)] = _AgChannel(depth_group, nbytes)
    e, parity, nbytes = ch.publish(w_shard.detach())
    staging = torch.empty((out_l, in_l), dtype=w_shard.dtype, device=a.device)
    ag = ch.context(e, parity, nbytes, staging, out_l // ch.n, n_copy=0)   # the launcher sets the CTA count
    ar_ref = None
    if ar_group is not None and dist.get_world_size(ar_group) > 1:
        arch = _channels.get(id(ar_group))
        if arch is None:
            arch = _channels[id(ar_group)] = _ArChannel(ar_group)
        bn, tiles = _tile_geometry(M, N)
        if layout == 0 and (out_l // ch.n) % 128:
            bn = 128
            tiles = (M + _BM - 1) // _BM * ((N + 127) // 128)
        arch.ensure(tiles, bn)
        ar_ctx = arch.context(bn)
        out, aux_t = _ar_outputs(arch, ar_ctx, (M, N), a.dtype, a.device, want_aux)
        ar_ref = ctypes.byref(ar_ctx)
    else:
        out = torch.empty((M, N), dtype=a.dtype, device=a.device)
        aux_t = torch.empty((M, N), dtype=a.dtype, device=a.device) if want_aux else None
    st = _lib.lib().axb_ag_gemm(
        ctypes.c_int(layout), _lib.ptr(a), _lib.ptr(out), _lib.ptr(bias), _lib.ptr(aux_t), ctypes.c_int(M),
        ctypes.c_int(N), ctypes.c_int(K), ctypes.c_int(_DT[a.dtype]), ctypes.c_int(_DT[out.dtype]),
        ctypes.c_int(epilogue), ctypes.c_int(a.device.index), _lib.stream_ptr(), ctypes.byref(ag), ar_ref)
    _lib.check(st, "axb_ag_gemm")
    return (out, staging, aux_t) if want_aux else (out, staging)


class AxbCommCtx(ctypes.Structure):
    _fields_ = [("n", ctypes.c_int), ("rank", ctypes.c_int), ("epoch", ctypes.c_uint), ("pad", ctypes.c_int),
                ("buf_peer", ctypes.c_void_p * 8), ("wait_local", ctypes.c_void_p),
                ("signal_peer", ctypes.c_void_p * 8), ("counter", ctypes.c_void_p)]


class _GradChannel:
    """Symmetric bucket + flags of the peer-memory gradient all-reduce for one group.
    Control block: READY[n] at 0, DONE[n] at 64, CTA counter at 256; the bucket starts at 4096."""

    _READY, _DONE, _COUNTER = 0, 64, 256

    def __init__(self, group, nbytes):
        self.group, self.n, self.rank = group, dist.get_world_size(group), dist.get_rank(group)
        self.capacity = (int(nbytes) + (1 << 22) - 1) // (1 << 22) * (1 << 22)
        torch.cuda.synchronize()
        self.buf = symm.SymmBuffer(group, _CTRL_BYTES + self.capacity, "grad_ar")
        self.buf.local.zero_()
        torch.cuda.synchronize()
        self.buf.barrier()
        dist.barrier(group=group)
        self.epoch = 0
        self.tables = {}

    def ctx(self, wait_off, signal_off):
        c = AxbCommCtx()
        c.n, c.rank, c.epoch = self.n, self.rank, self.epoch
        base = self.buf.peer_ptrs
        for j in range(self.n):
            c.buf_peer[j] = base[j] + _CTRL_BYTES
            c.signal_peer[j] = base[j] + signal_off
        c.wait_local = base[self.rank] + wait_off
        c.counter = base[self.rank] + self._COUNTER
        return c


_grad_channels = {}
_PK_CHUNK = 1 << 15


def _grad_table(ch, grads):
    key = tuple((g.data_ptr(), g.numel()) for g in grads)
    tab = ch.tables.get(key)
    if tab is None:
        rows, off, prefix = [], 0, 0
        for g in grads:
            rows.append((g.data_ptr(), g.numel(), 0, off, prefix))
            off += (g.numel() + 7) // 8 * 8
            prefix += (g.numel() + _PK_CHUNK - 1) // _PK_CHUNK
        dev_tab = torch.tensor(rows, dtype=torch.int64).to(grads[0].device)
        ch.tables.clear()
        tab = ch.tables[key] = (dev_tab, len(rows), prefix, off)
    return tab


class AxbGradArCtx(ctypes.Structure):
    _fields_ = [("n", ctypes.c_int), ("rank", ctypes.c_int), ("epoch", ctypes.c_uint), ("pad", ctypes.c_int),
                ("recv_peer", ctypes.c_void_p * 8), ("result_peer", ctypes.c_void_p * 8),
                ("pushed_local", ctypes.c_void_p), ("pushed_peer", ctypes.c_void_p * 8),
                ("reduced_local", ctypes.c_void_p), ("reduced_peer", ctypes.c_void_p * 8),
                ("counters", ctypes.c_void_p), ("slot_bytes", ctypes.c_ulonglong)]


class _GradArChannel:
    """Receive and result areas of the one-kernel gradient all-reduce for one group.
    Control block: PUSHED[n] at 0, REDUCED[n] at 64, counters at 256; then the receive area (n slots of
    ``slot_bytes``) and the result area (``result_bytes``)."""

    _PUSHED, _REDUCED, _COUNTERS = 0, 64, 256

    def __init__(self, group, slot_bytes, result_bytes):
        self.group, self.n, self.rank = group, dist.get_world_size(group), dist.get_rank(group)
        self.slot_bytes = (int(slot_bytes) + (1 << 20) - 1) // (1 << 20) * (1 << 20)
        self.result_bytes = (int(result_bytes) + (1 << 20) - 1) // (1 << 20) * (1 << 20)
        torch.cuda.synchronize()
        self.buf = symm.SymmBuffer(group, _CTRL_BYTES + self.n * self.slot_bytes + self.result_bytes, "grad_allreduce")
        self.buf.local[:_CTRL_BYTES].zero_()
        torch.cuda.synchronize()
        self.buf.barrier()
        dist.barrier(group=group)
        self.epoch = 0
        self.tables = {}

    def ctx(self):
        self.epoch += 1
        c = AxbGradArCtx()
        c.n, c.rank, c.epoch = self.n, self.rank, self.epoch
        base = self.buf.peer_ptrs
        for j in range(self.n):
            c.recv_peer[j] = base[j] + _CTRL_BYTES
            c.result_peer[j] = base[j] + _CTRL_BYTES + self.n * self.slot_bytes
            c.pushed_peer[j] = base[j] + self._PUSHED
            c.reduced_peer[j] = base[j] + self._REDUCED
        c.pushed_local = base[self.rank] + self._PUSHED
        c.reduced_local = base[self.rank] + self._REDUCED
        c.counters = base[self.rank] + self._COUNTERS
        c.slot_bytes = self.slot_bytes
        return c


_grad_ar_channels = {}
_GRAD_AR_MAX_BYTES = 512 << 20     # tensors of one call; longer lists are processed in several calls


def _grad_allreduce_one_kernel(grads, group, scale) -> None:
    """``csrc/allreduce.cu::grad_allreduce_kernel`` over ``grads`` (same dtype, contiguous)."""
    dtype = grads[0].dtype
    es = grads[0].element_size()
    n = dist.get_world_size(group)
    chunks = sum((g.numel() + _PK_CHUNK - 1) // _PK_CHUNK for g in grads)
    cps = (chunks + n - 1) // n
    slot_bytes, result_bytes = cps * _PK_CHUNK * es, chunks * _PK_CHUNK * es
    ch = _grad_ar_channels.get(id(group))
    if ch is None or ch.slot_bytes < slot_bytes or ch.result_bytes < result_bytes:
        ch = _grad_ar_channels[id(group)] = _GradArChannel(group, max(slot_bytes, 32 << 20),
                                                             max(result_bytes, n * (32 << 20)))
    key = tuple((g.data_ptr(), g.numel()) for g in grads)
    tab = ch.tables.get(key)
    if tab is None:
        rows, prefix = [], 0
        for g in grads:
            rows.append((g.data_ptr(), g.numel(), 0, 0, prefix))
            prefix += (g.numel() + _PK_CHUNK - 1) // _PK_CHUNK
        if len(ch.tables) > 8:
            ch.tables.clear()
        tab = ch.tables[key] = torch.tensor(rows, dtype=torch.int64).to(grads[0].device)
    ctx = ch.ctx()
    st = _lib.lib().axb_grad_allreduce(
        _lib.ptr(tab), ctypes.c_int(len(grads)), ctypes.c_longlong(chunks), ctypes.c_longlong(cps),
        ctypes.c_int(0 if dtype == torch.float32 else 1), ctypes.c_float(1.0 if scale is None else float(scale)),
        ctypes.byref(ctx), ctypes.c_int(grads[0].device.index), _lib.stream_ptr())
    _lib.check(st, "axb_grad_allreduce")


def try_all_reduce_scale_(grads, group, scale) -> bool:
    """Sum ``grads`` over ``group`` and multiply by ``scale`` with the peer-memory kernels: by default one
    kernel that reads and writes the gradient tensors directly (owners of the slices receive the partials,
    reduce in rank order, scale and hand the result to every peer); ``AXONN_GRAD_AR=bucket`` selects the older
    pack -> two-shot -> unpack form and ``AXONN_GRAD_AR=nvls`` the same with the reduction done inside the
    NVSwitch (``multimem.ld_reduce`` / ``multimem.st``; needs a multicast-bound symmetric allocation, i.e. NVLS
    not disabled for symmetric memory).  Returns False when not applicable."""
    if not grads or not group_usable(group, grads[0]):
        return False
    dtype = grads[0].dtype
    if dtype not in (torch.float32, torch.bfloat16) or any(g.dtype != dtype or not g.is_contiguous() for g in grads):
        return False
    import os

    mode = os.environ.get("AXONN_GRAD_AR", "fused")
    if mode not in ("bucket", "nvls"):
        es = grads[0].element_size()
        batch, size = [], 0
        for g in grads:
            padded = (g.numel() + _PK_CHUNK - 1) // _PK_CHUNK * _PK_CHUNK * es
            if batch and size + padded > _GRAD_AR_MAX_BYTES:
                _grad_allreduce_one_kernel(batch, group, scale)
                batch, size = [], 0
            batch.append(g)
            size += padded
        if batch:
            _grad_allreduce_one_kernel(batch, group, scale)
        return True
    es = 4 if dtype == torch.float32 else 2
    total_elems = sum((g.numel() + 7) // 8 * 8 for g in grads)
    n = dist.get_world_size(group)
    nbytes = (total_elems * es + 16 * n - 1) // (16 * n) * (16 * n)
    ch = _grad_channels.get(id(group))
    if ch is None or ch.capacity < nbytes:
        ch = _grad_channels[id(group)] = _GradChannel(group, nbytes)
    tab, ntens, chunks, _ = _grad_table(ch, grads)
    L = _lib.lib()
    dev = grads[0].device.index
    code = 0 if dtype == torch.float32 else 1
    bucket = ch.buf.peer_ptrs[ch.rank] + _CTRL_BYTES
    ch.epoch += 1
    pack = ch.ctx(ch._DONE, ch._READY)      # publishes READY
    _lib.check(L.axb_bucket_copy(_lib.ptr(tab), ctypes.c_int(ntens), ctypes.c_longlong(chunks),
                                 ctypes.c_void_p(bucket), ctypes.c_int(code), ctypes.c_int(0), ctypes.byref(pack),
                                 ctypes.c_int(dev), _lib.stream_ptr()), "axb_bucket_copy")
    red = ch.ctx(ch._READY, ch._DONE)       # waits READY, publishes DONE
    if mode == "nvls" and ch.buf.multicast_ptr:
        # reduction inside the NVSwitch: multimem.ld_reduce / multimem.st on the bucket's multicast address
        _lib.check(L.axb_allreduce_nvls(ctypes.c_longlong(nbytes), ctypes.c_int(code),
                                        ctypes.c_float(1.0 if scale is None else float(scale)),
                                        ctypes.c_void_p(ch.buf.multicast_ptr + _CTRL_BYTES), ctypes.byref(red),
                                        ctypes.c_int(dev), _lib.stream_ptr()), "axb_allreduce_nvls")
    else:
        _lib.check(L.axb_allreduce_twoshot(ctypes.c_longlong(nbytes), ctypes.c_int(code),
                                           ctypes.c_float(1.0 if scale is None else float(scale)), ctypes.byref(red),
                                           ctypes.c_int(dev), _lib.stream_ptr()), "axb_allreduce_twoshot")
    unpack = ch.ctx(ch._DONE, ch._READY)    # waits DONE
    _lib.check(L.axb_bucket_copy(_lib.ptr(tab), ctypes.c_int(ntens), ctypes.c_longlong(chunks),
                                 ctypes.c_void_p(bucket), ctypes.c_int(code), ctypes.c_int(1), ctypes.byref(unpack),
                                 ctypes.c_int(dev), _lib.stream_ptr()), "axb_bucket_copy")
    return True


# ----------------------------------------------------------------------------- row all-to-all / embedding rows
class AxbP2pCtx(ctypes.Structure):
    _fields_ = [("n", ctypes.c_int), ("rank", ctypes.c_int), ("epoch", ctypes.c_uint), ("pad", ctypes.c_int),
                ("base_peer", ctypes.c_void_p * 8), ("mail_local", ctypes.c_void_p),
                ("mail_peer", ctypes.c_void_p * 8), ("done_local", ctypes.c_void_p),
                ("done_peer", ctypes.c_void_p * 8), ("counter", ctypes.c_void_p), ("out_off", ctypes.c_ulonglong)]


class AxbRowBlock(ctypes.Structure):
    _fields_ = [("src", ctypes.c_void_p), ("src_pitch", ctypes.c_longlong), ("dst_off", ctypes.c_longlong),
                ("dst_pitch", ctypes.c_longlong), ("rows", ctypes.c_longlong), ("row_bytes", ctypes.c_longlong)]


class _P2pChannel:
    """Control words (and optionally a data region) of the row all-to-all / embedding kernels for one group.
    Layout: mailbox (n records of 32 bytes) at 0, DONE[n] at 512, CTA counters at 1024, data from 4096."""

    _MAIL, _DONE, _COUNTER = 0, 512, 1024

    def __init__(self, group, data_bytes=0, tag="p2p"):
        self.group, self.n, self.rank = group, dist.get_world_size(group), dist.get_rank(group)
        self.data_bytes = (int(data_bytes) + 255) // 256 * 256
        torch.cuda.synchronize()
        self.buf = symm.SymmBuffer(group, _CTRL_BYTES + self.data_bytes, tag)
        self.buf.local.zero_()
        torch.cuda.synchronize()
        self.buf.barrier()
        dist.barrier(group=group)
        self.epoch = 0

    def ctx(self, base_peer, out_off=0):
        self.epoch += 1
        base = self.buf.peer_ptrs
        c = AxbP2pCtx()
        c.n, c.rank, c.epoch = self.n, self.rank, self.epoch
        for j in range(self.n):
            c.base_peer[j] = base_peer[j]
            c.mail_peer[j] = base[j] + self._MAIL
            c.done_peer[j] = base[j] + self._DONE
        c.mail_local = base[self.rank] + self._MAIL
        c.done_local = base[self.rank] + self._DONE
        c.counter = base[self.rank] + self._COUNTER
        c.out_off = out_off
        return c

    def data_ptrs(self):
        return [p + _CTRL_BYTES for p in self.buf.peer_ptrs]

    def data_view(self, dtype, numel):
        return self.buf.view(dtype, numel, _CTRL_BYTES)


_a2a_channels = {}


def a2a_rows_usable(group, tensor) -> bool:
    return group_usable(group, tensor) and symm.output_arena() is not None


def a2a_rows(group, blocks, out_shape, dtype, device):
    """All-to-all-v of row blocks in one kernel (``csrc/p2p.cu``): ``blocks[j]`` = ``(src_ptr, src_pitch,
    dst_off, dst_pitch, rows, row_bytes)`` describes what this rank stores into rank ``j``'s output (byte
    quantities, multiples of 16).  The output tensor of shape ``out_shape`` is allocated from the peer-mapped
    arena and returned complete (the kernel ends after every peer has finished storing into it)."""
    arena = symm.output_arena()
    ch = _a2a_channels.get(id(group))
    if ch is None:
        ch = _a2a_channels[id(group)] = _P2pChannel(group, 0, "a2a_rows")
    out = arena.empty(out_shape, dtype)
    ctx = ch.ctx(arena.peer_bases(group), arena.offset(out))
    arr = (AxbRowBlock * ch.n)()
    for j, (src, sp, doff, dp, rows, rb) in enumerate(blocks):
        arr[j].src, arr[j].src_pitch, arr[j].dst_off, arr[j].dst_pitch, arr[j].rows, arr[j].row_bytes = \
            src, sp, doff, dp, rows, rb
    st = _lib.lib().axb_a2a_rows(ctypes.byref(ctx), arr, ctypes.c_int(device.index), _lib.stream_ptr())
    _lib.check(st, "axb_a2a_rows")
    return out


class _EmbeddingChannel:
    """Peer-mapped copies of the depth shards of an embedding table (forward) and fp32 gradient shards
    (backward) for one depth group."""

    def __init__(self, group, shard_bytes, grad_bytes):
        self.fwd = _P2pChannel(group, shard_bytes, "embedding_rows")
        self.bwd = _P2pChannel(group, grad_bytes, "embedding_grad")
        self.shard_bytes, self.grad_bytes = shard_bytes, grad_bytes


_emb_channels = {}


def embedding_p2p_usable(group, table_shard, rows_per_shard, row_elems) -> bool:
    return (table_shard.dtype == torch.bfloat16 and group_usable(group, table_shard)
            and (row_elems * 2) % 16 == 0 and table_shard.numel() == rows_per_shard * row_elems)


def _emb_channel(group, shard):
    nbytes = shard.numel() * shard.element_size()
    gbytes = shard.numel() * 4
    ch = _emb_channels.get(id(group))
    if ch is None or ch.shard_bytes < nbytes or ch.grad_bytes < gbytes:
        ch = _emb_channels[id(group)] = _EmbeddingChannel(group, nbytes, gbytes)
    return ch


def embedding_fetch(group, ids, table_shard, rows_per_shard, row_elems):
    """Rows ``ids`` of a table whose row blocks are sharded over ``group``: every token's row is fetched from
    the owning rank's published shard over NVLink; the table is never gathered.  ``ids`` int64 ``[T]``;
    returns bf16 ``[T, row_elems]``."""
    ch = _emb_channel(group, table_shard).fwd
    L = _lib.lib()
    dev = table_shard.device
    # publish my shard: copy into the peer-mapped buffer, then raise this call's epoch in every peer's mailbox
    ctx = ch.ctx(ch.data_ptrs())
    ch.data_view(torch.bfloat16, table_shard.numel()).copy_(table_shard.detach().reshape(-1))
    _lib.check(L.axb_p2p_publish(ctypes.byref(ctx), ctypes.c_int(dev.index), _lib.stream_ptr()), "axb_p2p_publish")
    ids = ids.reshape(-1).contiguous()
    out = torch.empty((ids.numel(), row_elems), dtype=torch.bfloat16, device=dev)
    st = L.axb_embedding_fetch(_lib.ptr(ids), ctypes.c_longlong(ids.numel()), _lib.ptr(out),
                               ctypes.c_longlong(row_elems * 2), ctypes.c_longlong(rows_per_shard),
                               ctypes.byref(ctx), ctypes.c_int(dev.index), _lib.stream_ptr())
    _lib.check(st, "axb_embedding_fetch")
    return out


def embedding_scatter_add(group, ids, dy, rows_per_shard, row_elems, shard_numel):
    """Gradient of ``embedding_fetch`` w.r.t. the table: every token's gradient row is added into the owning
    rank's fp32 gradient shard with remote atomics; returns this rank's summed shard (fp32, flat)."""
    ch_all = _emb_channels[id(group)]
    ch = ch_all.bwd
    L = _lib.lib()
    dev = dy.device
    ctx = ch.ctx(ch.data_ptrs())
    grad = ch.data_view(torch.float32, shard_numel)
    grad.zero_()
    _lib.check(L.axb_p2p_publish(ctypes.byref(ctx), ctypes.c_int(dev.index), _lib.stream_ptr()), "axb_p2p_publish")
    ids = ids.reshape(-1).contiguous()
    dy = dy.reshape(-1, row_elems).contiguous()
    st = L.axb_embedding_scatter_add(_lib.ptr(ids), ctypes.c_longlong(ids.numel()), _lib.ptr(dy),
                                     ctypes.c_int(row_elems), ctypes.c_longlong(rows_per_shard), ctypes.byref(ctx),
                                     ctypes.c_int(dev.index), _lib.stream_ptr())
    _lib.check(st, "axb_embedding_scatter_add")
    return grad.clone()
