"""Sequence parallelism for long contexts: every rank of a group holds a slice of the sequence.

The reference never splits the sequence dimension (no ring attention, context parallelism or all-to-all
attention anywhere in ``axonn/``); what bounds its context length is the activation memory of one whole sequence
per rank.  Here the ranks of a *sequence group* - by default the data-parallel group, whose ranks hold the same
weights - each take ``S / n`` consecutive tokens of the same samples.  Everything that works token by token
(embeddings, norms, the feed-forward layers, the loss) runs on the slice unchanged; attention exchanges the
slices for heads with two all-to-alls (the DeepSpeed-Ulysses scheme):

    [B, S/n, all local heads]  --all-to-all-->  [B, S, local heads / n]  --attention-->  --all-to-all-->  back

Rotary embeddings are applied between the first exchange and the attention, where a rank sees whole sequences,
so they need no position offset; learned position embeddings are looked up at ``rank * S/n + i``.  Gradients of
the (replicated) weights are summed over the sequence group by the ordinary data-parallel gradient
synchronisation: with equal slices, the mean over ranks of the per-slice mean losses is the mean over all tokens.

Activation memory per rank falls by ``n``; the price is two all-to-alls of the attention input and output per
layer and direction.  The number of local key/value heads (after row tensor parallelism) must be a multiple of
``n``.
"""

from typing import Optional

import torch
import torch.distributed as dist

from .. import axonn as ax
from .. import ops


class _SeqAllToAll(torch.autograd.Function):
    """Split ``x`` along ``scatter_dim`` over the group and concatenate what arrives along ``gather_dim`` (rank
    order).  Its backward is the same exchange with the two dimensions swapped."""

    @staticmethod
    def forward(ctx, x, group, scatter_dim, gather_dim):
        ctx.group, ctx.scatter_dim, ctx.gather_dim = group, scatter_dim, gather_dim
        n = dist.get_world_size(group)
        if n == 1:
            return x
        if x.shape[scatter_dim] % n:
            raise ValueError(f"dimension {scatter_dim} of size {x.shape[scatter_dim]} does not split over {n} ranks")
        send = torch.stack(x.chunk(n, dim=scatter_dim), 0).contiguous()       # [n, ...]: piece j goes to rank j
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send, group=group)
        return torch.cat(recv.unbind(0), dim=gather_dim)                      # piece j came from rank j

    @staticmethod
    def backward(ctx, grad):
        return _SeqAllToAll.apply(grad.contiguous(), ctx.group, ctx.gather_dim, ctx.scatter_dim), None, None, None


def seq_all_to_all(x, group, scatter_dim: int, gather_dim: int):
    return _SeqAllToAll.apply(x, group, scatter_dim, gather_dim)


def ulysses_attention_packed(qkv, group, rope=None, causal=True):
    """Causal attention on a packed projection ``[B, S/n, kv_groups, q_per_kv + 2, D]`` whose sequence is split over
    ``group`` in rank order.  ``rope`` (optional) is applied to the exchanged tensor ``[B, S, kv_groups / n, ...]``,
    i.e. on whole sequences.  Returns ``[B, S/n, kv_groups * q_per_kv, D]``."""
    x = seq_all_to_all(qkv, group, scatter_dim=2, gather_dim=1)
    if rope is not None:
        x = rope(x)
    o = ops.flash_attention_packed(x, causal=causal)
    return seq_all_to_all(o, group, scatter_dim=1, gather_dim=2)


def shard_sequence(t, group=None, dim: int = 1):
    """This rank's slice of ``t`` along the sequence dimension (``group`` defaults to the data-parallel group)."""
    group = ax.comm_handle.data_parallel_group if group is None else group
    n, me = dist.get_world_size(group), dist.get_rank(group)
    if t.shape[dim] % n:
        raise ValueError(f"sequence length {t.shape[dim]} does not split over {n} ranks")
    per = t.shape[dim] // n
    return t.narrow(dim, me * per, per).contiguous()


def enable_sequence_parallel(model, group: Optional[object] = None):
    """Switch ``model`` (one of this package's transformer models, or anything built from ``ParallelAttention``) to
    sequence parallelism over ``group`` (default: the data-parallel group).  Afterwards the model expects token and
    target tensors that hold this rank's slice of every sequence (``shard_sequence``), and every rank of the group
    must be given the same samples.  Returns the model."""
    from ..models.blocks import ParallelAttention

    group = ax.comm_handle.data_parallel_group if group is None else group
    n = dist.get_world_size(group)
    found = 0
    for m in model.modules():
        if isinstance(m, ParallelAttention):
            if m.groups_l % n:
                raise ValueError(f"{m.groups_l} local key/value heads do not split over {n} sequence-parallel ranks")
            m.sequence_group = group if n > 1 else None
            found += 1
    if not found:
        raise ValueError("the model has no ParallelAttention layer")
    if hasattr(model, "sequence_group"):
        model.sequence_group = group if n > 1 else None       # learned positions need the slice's offset
    return model
