"""Layout switches between pure data parallelism and 3-D tensor parallelism.

In "easy mode" (``expert_mode=False``) every rank feeds a tensor-parallel
layer its own batch shard ``[m_i, k]`` with all ``k`` features.  The layer
needs ``[sum m_i, k/G]`` instead, and hands back ``[m_i, n]`` afterwards.  These
are the operators that move between the two layouts; they correspond to the
reference's ``axonn/intra_layer/asym_communication.py:16-252``
(``gather_batch_sizes``, ``Gatherv``/``Dropv``,
``GatherBatchScatterChannels``/``GatherChannelsScatterBatch``).

Differences: row counts are exchanged once per distinct (group, local rows)
pair and cached on the host, so steady-state steps have no device-to-host
synchronisation (the reference syncs twice per layer call, ``:16-30``).  On
GPUs whose group shares peer memory each exchange is one kernel
(``csrc/p2p.cu::a2a_rows_kernel``) in which every rank stores its row blocks
straight into the destination's output tensor over NVLink - the transposition
is done by the addressing, without the pack / unpack copies around a library
all-to-all.  Elsewhere (CPU ranks, ``AXONN_BACKEND=nccl``) the exchanges are
single ``all_to_all_single`` / ``all_gather`` calls on contiguous buffers.
"""

from typing import List

import torch
import torch.distributed as dist

from .. import axonn as ax

_batch_size_cache = {}


def clear_batch_size_cache():
    _batch_size_cache.clear()


@torch.no_grad()
def gather_batch_sizes(local_batch_size: int, process_group=None, device=None) -> torch.Tensor:
    """Row count of every rank of ``process_group`` as a CPU int64 tensor.

    The answer is cached per (group, local row count): ranks of a group change
    their batch size together in every supported data pipeline
    (``drop_last=True``).  ``clear_batch_size_cache()`` drops the cache."""
    n = dist.get_world_size(process_group)
    if n == 1:
        return torch.tensor([int(local_batch_size)], dtype=torch.int64)
    key = (id(process_group), int(local_batch_size))
    hit = _batch_size_cache.get(key)
    if hit is not None:
        return hit
    t = ax.get_timers()
    t.start("gather-batch-sizes")
    if device is None:
        device = ax.comm_handle.device if ax.comm_handle is not None else "cpu"
    mine = torch.tensor([int(local_batch_size)], dtype=torch.int64, device=device)
    everyone = torch.empty(n, dtype=torch.int64, device=device)
    dist.all_gather_into_tensor(everyone, mine, group=process_group)
    everyone = everyone.cpu()
    t.stop("gather-batch-sizes")
    _batch_size_cache[key] = everyone
    return everyone


def _p2p_ok(tensor, process_group, row_bytes) -> bool:
    """The peer-memory row all-to-all applies: CUDA tensor, peer-capable group, 16-byte row granularity."""
    if not tensor.is_cuda or row_bytes % 16 or tensor.data_ptr() % 16:
        return False
    from ..parallel import fused

    return fused.a2a_rows_usable(process_group, tensor)


def _sizes(rank_local_batch_sizes) -> List[int]:
    if isinstance(rank_local_batch_sizes, torch.Tensor):
        return [int(v) for v in rank_local_batch_sizes.tolist()]
    return [int(v) for v in rank_local_batch_sizes]


@torch.no_grad()
def _allgatherv(tensor, rank_local_batch_sizes, process_group=None):
    """Concatenate row blocks of unequal height from every rank."""
    sizes = _sizes(rank_local_batch_sizes)
    n = dist.get_world_size(process_group)
    if n == 1:
        return tensor
    t = ax.get_timers()
    t.start("allgatherv")
    tensor = tensor.contiguous()
    tail = tuple(tensor.shape[1:])
    row_bytes = tensor.element_size()
    for t_ in tail:
        row_bytes *= t_
    if _p2p_ok(tensor, process_group, row_bytes):
        from ..parallel import fused

        me = dist.get_rank(process_group)
        off = sum(sizes[:me]) * row_bytes
        blocks = [(tensor.data_ptr(), row_bytes, off, row_bytes, tensor.shape[0], row_bytes)] * n
        out = fused.a2a_rows(process_group, blocks, (sum(sizes),) + tail, tensor.dtype, tensor.device)
        t.stop("allgatherv")
        return out
    out = torch.empty((sum(sizes),) + tail, dtype=tensor.dtype, device=tensor.device)
    if len(set(sizes)) == 1:
        dist.all_gather_into_tensor(out, tensor, group=process_group)
    elif tensor.is_cuda:
        # unequal heights: an all-to-all whose sends are all the same block
        outs = list(torch.split(out, sizes, dim=0))
        dist.all_to_all(outs, [tensor for _ in range(n)], group=process_group)
    else:
        # the same exchange through the single-tensor form (gloo has no list all-to-all): the block is sent once
        # per rank out of an n-fold copy
        m = tensor.shape[0]
        send = tensor.unsqueeze(0).expand((n,) + tuple(tensor.shape)).reshape((n * m,) + tail)
        dist.all_to_all_single(out, send.contiguous(), output_split_sizes=sizes, input_split_sizes=[m] * n,
                               group=process_group)
    t.stop("allgatherv")
    return out


def _my_rows(rank_local_batch_sizes, process_group):
    sizes = _sizes(rank_local_batch_sizes)
    me = dist.get_rank(process_group)
    start = sum(sizes[:me])
    return start, start + sizes[me]


class Gatherv(torch.autograd.Function):
    """forward: ``[m_i, k] -> [sum m_i, k]``; backward: keep my rows."""

    @staticmethod
    def forward(ctx, input_, rank_local_batch_sizes, process_group=None):
        t = ax.get_timers()
        t.start("extra-non-expert-communication")
        out = _allgatherv(input_, rank_local_batch_sizes, process_group)
        ctx.sizes, ctx.process_group = rank_local_batch_sizes, process_group
        t.stop("extra-non-expert-communication")
        return out.view_as(out) if out is input_ else out

    @staticmethod
    def backward(ctx, grad_output):
        a, b = _my_rows(ctx.sizes, ctx.process_group)
        return grad_output[a:b], None, None


class Dropv(torch.autograd.Function):
    """forward: keep my rows of ``[sum m_i, k]``; backward: all-gather-v."""

    @staticmethod
    def forward(ctx, input_, rank_local_batch_sizes, process_group=None):
        a, b = _my_rows(rank_local_batch_sizes, process_group)
        ctx.sizes, ctx.process_group = rank_local_batch_sizes, process_group
        return input_[a:b]

    @staticmethod
    def backward(ctx, grad_output):
        t = ax.get_timers()
        t.start("extra-non-expert-communication")
        g = _allgatherv(grad_output, ctx.sizes, ctx.process_group)
        t.stop("extra-non-expert-communication")
        return g, None, None


@torch.no_grad()
def _gather_batch_scatter_channels(input_, rank_local_batch_sizes, process_group=None):
    """``[m_i, k]`` on rank i  ->  ``[sum m_i, k/G]`` (my feature chunk of everyone's rows)."""
    n = dist.get_world_size(process_group)
    if n == 1:
        return input_
    sizes = _sizes(rank_local_batch_sizes)
    t = ax.get_timers()
    t.start("gather-batch-scatter-channels")
    t.start("alltoallv")
    m, k = input_.shape[0], input_.shape[-1]
    if k % n != 0:
        raise ValueError(f"feature dim {k} not divisible by group size {n}")
    es = input_.element_size()
    if input_.ndim == 2 and _p2p_ok(input_, process_group, (k // n) * es):
        # rank j receives my columns [j*k/G, (j+1)*k/G) of all my rows, at the rows of my batch offset
        from ..parallel import fused

        x = input_.contiguous()
        me, kc = dist.get_rank(process_group), k // n
        off = sum(sizes[:me]) * kc * es
        blocks = [(x.data_ptr() + j * kc * es, k * es, off, kc * es, m, kc * es) for j in range(n)]
        recv = fused.a2a_rows(process_group, blocks, (sum(sizes), kc), x.dtype, x.device)
        t.stop("alltoallv")
        t.stop("gather-batch-scatter-channels")
        return recv
    # [m, G, k/G] -> [G, m, k/G]: chunk j goes to rank j
    send = input_.reshape(m, n, k // n).transpose(0, 1).contiguous()
    recv = torch.empty((sum(sizes), k // n), dtype=input_.dtype, device=input_.device)
    dist.all_to_all_single(
        recv, send.reshape(n * m, k // n), output_split_sizes=sizes, input_split_sizes=[m] * n, group=process_group
    )
    t.stop("alltoallv")
    t.stop("gather-batch-scatter-channels")
    return recv


@torch.no_grad()
def _gather_channels_scatter_batch(input_, rank_local_batch_sizes, process_group=None):
    """``[sum m_i, k/G]`` -> ``[m_me, k]`` (all feature chunks of my rows)."""
    n = dist.get_world_size(process_group)
    if n == 1:
        return input_
    sizes = _sizes(rank_local_batch_sizes)
    me = dist.get_rank(process_group)
    t = ax.get_timers()
    t.start("gather-channels-scatter-batch")
    t.start("alltoallv")
    input_ = input_.contiguous()
    kc = input_.shape[-1]
    mine = sizes[me]
    es = input_.element_size()
    if input_.ndim == 2 and _p2p_ok(input_, process_group, kc * es):
        # rank j receives my feature chunk of ITS rows, at column block `me` of its [m_j, G * kc] output
        from ..parallel import fused

        blocks, start = [], 0
        for j in range(n):
            blocks.append((input_.data_ptr() + start * kc * es, kc * es, me * kc * es, n * kc * es, sizes[j], kc * es))
            start += sizes[j]
        out = fused.a2a_rows(process_group, blocks, (mine, n * kc), input_.dtype, input_.device)
        t.stop("alltoallv")
        t.stop("gather-channels-scatter-batch")
        return out
    recv = torch.empty((n * mine, kc), dtype=input_.dtype, device=input_.device)
    dist.all_to_all_single(
        recv, input_, output_split_sizes=[mine] * n, input_split_sizes=sizes, group=process_group
    )
    out = recv.reshape(n, mine, kc).transpose(0, 1).reshape(mine, n * kc)
    t.stop("alltoallv")
    t.stop("gather-channels-scatter-batch")
    return out


class GatherBatchScatterChannels(torch.autograd.Function):
    @staticmethod
    def forward(ctx, input_, rank_local_batch_sizes, process_group=None):
        t = ax.get_timers()
        t.start("extra-non-expert-communication")
        out = _gather_batch_scatter_channels(input_, rank_local_batch_sizes, process_group)
        ctx.sizes, ctx.process_group = rank_local_batch_sizes, process_group
        t.stop("extra-non-expert-communication")
        return out.view_as(out) if out is input_ else out

    @staticmethod
    def backward(ctx, grad_output):
        t = ax.get_timers()
        t.start("extra-non-expert-communication")
        g = _gather_channels_scatter_batch(grad_output, ctx.sizes, ctx.process_group)
        t.stop("extra-non-expert-communication")
        return g, None, None


class GatherChannelsScatterBatch(torch.autograd.Function):
    @staticmethod
    def forward(ctx, input_, rank_local_batch_sizes, process_group=None):
        t = ax.get_timers()
        t.start("extra-non-expert-communication")
        out = _gather_channels_scatter_batch(input_, rank_local_batch_sizes, process_group)
        ctx.sizes, ctx.process_group = rank_local_batch_sizes, process_group
        t.stop("extra-non-expert-communication")
        return out.view_as(out) if out is input_ else out

    @staticmethod
    def backward(ctx, grad_output):
        t = ax.get_timers()
        t.start("extra-non-expert-communication")
        g = _gather_batch_scatter_channels(grad_output, ctx.sizes, ctx.process_group)
        t.stop("extra-non-expert-communication")
        return g, None, None
