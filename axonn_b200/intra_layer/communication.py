"""Collective primitives and their autograd pairs for tensor parallelism.

Same operator set as the reference's ``axonn/intra_layer/communication.py``
(``_all_reduce``, ``_drop``, ``_gather``, ``_reduce_scatter`` and the autograd
Functions ``ForwardAllReduce``, ``BackwardAllReduce``, ``Drop``, ``Gather``,
``ForwardGather_BackwardReduceScatter``).  The collectives write straight into
their final layout: gathering along a non-leading dimension uses one
``all_gather_into_tensor`` plus a single strided copy instead of a list gather
followed by ``cat`` + ``contiguous`` (reference ``:49-60``).
"""

import torch
import torch.distributed as dist

from . import overlap_communication as oc


def _size(group):
    return dist.get_world_size(group)


def _all_reduce(input_, process_group=None, overlap_comm=False):
    input_ = input_.contiguous()
    if _size(process_group) > 1:
        h = dist.all_reduce(input_, group=process_group, async_op=overlap_comm)
        if overlap_comm:
            oc.register_handle(h)
    return input_


def _drop(input_, dim, process_group=None):
    """Keep this rank's chunk of ``input_`` along ``dim``."""
    n = _size(process_group)
    if n == 1:
        return input_
    me = dist.get_rank(process_group)
    if input_.shape[dim] % n != 0:
        raise ValueError(f"dim {dim} of size {input_.shape[dim]} is not divisible by group size {n}")
    chunk = input_.shape[dim] // n
    return torch.narrow(input_, dim, me * chunk, chunk)


def _p2p_rows_ok(tensor, process_group, row_bytes, out_bytes) -> bool:
    """The peer-memory row kernel can serve this exchange: CUDA, peer-capable group, 16-byte rows, and an output
    that is small against the output arena (a rule every rank evaluates identically, so all ranks of the group
    take the same path)."""
    if not tensor.is_cuda or row_bytes % 16 or tensor.data_ptr() % 16:
        return False
    from ..parallel import fused, symm

    arena = symm.output_arena()
    return arena is not None and out_bytes * 16 <= arena.nbytes and fused.a2a_rows_usable(process_group, tensor)


def _gather_raw(input_, dim, process_group):
    n = _size(process_group)
    input_ = input_.contiguous()
    dim = dim % input_.ndim
    # Peer-memory all-gather: every rank stores its block straight into its place in every rank's output
    # (rows = the dimensions before `dim`, one row = this rank's extent of `dim` and everything behind it), so
    # a gather along an inner dimension needs no concatenation copy afterwards.
    rows = 1
    for d_ in input_.shape[:dim]:
        rows *= d_
    row_bytes = input_.element_size()
    for d_ in input_.shape[dim:]:
        row_bytes *= d_
    if input_.numel() > 0 and _p2p_rows_ok(input_, process_group, row_bytes, n * rows * row_bytes):
        from ..parallel import fused

        me = dist.get_rank(process_group)
        shape = list(input_.shape)
        shape[dim] *= n
        blocks = [(input_.data_ptr(), row_bytes, me * row_bytes, n * row_bytes, rows, row_bytes)] * n
        return fused.a2a_rows(process_group, blocks, tuple(shape), input_.dtype, input_.device)
    flat = torch.empty((n * input_.shape[0],) + tuple(input_.shape[1:]), dtype=input_.dtype,
                       device=input_.device)
    dist.all_gather_into_tensor(flat, input_, group=process_group)
    if dim == 0:
        return flat
    stacked = flat.reshape((n,) + tuple(input_.shape))
    # [n, d0, .., dk, ..] -> [d0, .., n*dk, ..] with one copy
    out = stacked.movedim(0, dim)
    shape = list(input_.shape)
    shape[dim] *= n
    return out.reshape(shape)


def _gather(input_, dim, process_group=None, cache=False):
    """All-gather along ``dim``.  For flat weight shards the prefetch cache of
    ``overlap_communication`` is consulted first."""
    if _size(process_group) == 1:
        return input_
    key = id(input_)
    if key in oc.weights_cache and oc.weights_cache[key][0] is input_:
        output, handle = oc.retrieve_all_gathered_weight(input_, delete=not cache)
        if handle is not None:
            handle.wait()
            if cache:
                oc.weights_cache[key][2] = None
        return output
    output = _gather_raw(input_, dim, process_group)
    if cache:
        oc.weights_cache[key] = [input_, output, None]
    return output


def _reduce_scatter(input_, dim, process_group=None, overlap_comm=False):
    if dim != 0:
        raise NotImplementedError("reduce-scatter is implemented for dim 0")
    n = _size(process_group)
    if n == 1:
        return input_
    if input_.shape[0] % n != 0:
        raise ValueError("leading dim not divisible by group size")
    input_ = input_.contiguous()
    shape = list(input_.shape)
    shape[0] //= n
    shard_bytes = input_.numel() // n * input_.element_size()
    if input_.numel() > 0 and _p2p_rows_ok(input_, process_group, shard_bytes, n * shard_bytes):
        # Peer-memory reduce-scatter: chunk j of every rank is stored into slot [source rank] of rank j's
        # receive tensor in one kernel, then summed locally in rank order (fp32 accumulation)
        from ..parallel import fused

        me = dist.get_rank(process_group)
        blocks = [(input_.data_ptr() + j * shard_bytes, shard_bytes, me * shard_bytes, shard_bytes, 1, shard_bytes)
                  for j in range(n)]
        parts = fused.a2a_rows(process_group, blocks, (n,) + tuple(shape), input_.dtype, input_.device)
        return parts.sum(0, dtype=torch.float32).to(input_.dtype) if input_.dtype != torch.float32 else parts.sum(0)
    output = torch.empty(shape, dtype=input_.dtype, device=input_.device)
    h = dist.reduce_scatter_tensor(output, input_, group=process_group, async_op=overlap_comm)
    if overlap_comm:
        oc.register_handle(h)
        # keep the send buffer alive until the handle has been waited on
        oc.handles.append(_KeepAlive(input_))
    return output


class _KeepAlive:
    """Handle-shaped object that only pins a tensor until ``clear_handles``."""

    def __init__(self, t):
        self.t = t

    def wait(self):
        self.t = None


class ForwardAllReduce(torch.autograd.Function):
    """forward: all-reduce; backward: identity."""

    @staticmethod
    def forward(ctx, input_, process_group=None):
        return _all_reduce(input_.clone() if _size(process_group) > 1 else input_, process_group)

    @staticmethod
    def backward(ctx, grad_output):
        return grad_output, None


class BackwardAllReduce(torch.autograd.Function):
    """forward: identity; backward: all-reduce (optionally asynchronous with the
    result added to the input's ``.grad`` at ``optimize_communication`` exit)."""

    @staticmethod
    def forward(ctx, input_, process_group=None, overlap_comm=False):
        ctx.process_group = process_group
        ctx.overlap_comm = overlap_comm
        ctx.input = input_ if overlap_comm else None
        return input_.view_as(input_)

    @staticmethod
    def backward(ctx, grad_output):
        g = grad_output.clone() if _size(ctx.process_group) > 1 else grad_output
        grad_input = _all_reduce(g, ctx.process_group, ctx.overlap_comm)
        if not ctx.overlap_comm:
            return grad_input, None, None
        oc.accumulate_later(ctx.input, grad_input)
        return None, None, None


class Drop(torch.autograd.Function):
    """forward: keep my chunk along ``dim``; backward: all-gather."""

    @staticmethod
    def forward(ctx, input_, process_group=None, dim=-1):
        ctx.process_group, ctx.dim = process_group, dim
        return _drop(input_, dim=dim, process_group=process_group)

    @staticmethod
    def backward(ctx, grad_output):
        return _gather(grad_output, dim=ctx.dim, process_group=ctx.process_group), None, None


class Gather(torch.autograd.Function):
    """forward: all-gather along ``dim``; backward: keep my chunk (valid when the
    incoming gradient is identical on all ranks of the group)."""

    @staticmethod
    def forward(ctx, input_, process_group=None, dim=-1):
        ctx.process_group, ctx.dim = process_group, dim
        return _gather(input_, dim=dim, process_group=process_group)

    @staticmethod
    def backward(ctx, grad_output):
        return _drop(grad_output, dim=ctx.dim, process_group=ctx.process_group), None, None


class GatherSumBackward(torch.autograd.Function):
    """forward: all-gather along dim 0 over ``gather_group``; backward:
    reduce-scatter over ``gather_group`` and all-reduce over ``sum_group``.

    Used for biases of layers whose output lives in data-parallel layout: every
    rank of both groups adds the *same* gathered bias to a *different* batch
    shard, so the bias gradient is the sum over all of them.  (The reference
    uses a plain ``Gather`` there and loses those contributions; its bias tests
    are skipped, ``axonn/tests/test_intra_layer_fc.py:99-100``.)"""

    @staticmethod
    def forward(ctx, input_, gather_group, sum_group):
        ctx.gather_group, ctx.sum_group = gather_group, sum_group
        return _gather(input_, dim=0, process_group=gather_group)

    @staticmethod
    def backward(ctx, grad_output):
        g = grad_output.contiguous()
        if _size(ctx.sum_group) > 1:
            g = g.clone()
            dist.all_reduce(g, group=ctx.sum_group)
        g = _reduce_scatter(g, 0, ctx.gather_group)
        return g, None, None


class ForwardGather_BackwardReduceScatter(torch.autograd.Function):
    """forward: all-gather along dim 0 (depth gather of a flat weight);
    backward: reduce-scatter, optionally asynchronous with deferred ``.grad``
    accumulation."""

    @staticmethod
    def forward(ctx, input_, process_group=None, dim=0, overlap_comm=False, cache_all_gather=False):
        assert dim == 0
        ctx.process_group, ctx.dim, ctx.overlap_comm = process_group, dim, overlap_comm
        ctx.input = input_
        out = _gather(input_, dim=dim, process_group=process_group, cache=cache_all_gather)
        return out.view_as(out) if out is input_ else out

    @staticmethod
    def backward(ctx, grad_output):
        grad_input = _reduce_scatter(
            grad_output, dim=ctx.dim, process_group=ctx.process_group, overlap_comm=ctx.overlap_comm
        )
        if not ctx.overlap_comm or _size(ctx.process_group) == 1:
            return grad_input, None, None, None, None
        oc.accumulate_later(ctx.input, grad_input)
        return None, None, None, None, None
