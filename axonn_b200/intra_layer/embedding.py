"""Tensor-parallel ``Embedding``.

Counterpart of the reference's ``axonn/intra_layer/embedding.py:57-222``: the
table is kept as ``[V, H]`` with ``H`` split over the outer group (inner group
when ``transpose``), flattened and depth-sharded; the other group must have
size one.  Forward gathers the table over depth, looks rows up and, in easy
mode, gathers the hidden dimension back.

On GPUs whose depth group shares peer memory the table is never gathered:
every token fetches its row from the depth rank that owns it, and the backward
adds the token gradients into the owners' gradient shards with remote atomics
(``csrc/p2p.cu``; ``AXONN_EMBEDDING_P2P=0`` keeps the gather).  For a 128256 x
4096 table that replaces 1 GB of all-gather per forward and a 1 GB
reduce-scatter per backward by the rows actually used.
"""

import torch
import torch.distributed as dist
import torch.nn.functional as F

from .. import axonn as ax
from ..utils import divide
from .communication import ForwardGather_BackwardReduceScatter, Gather, _gather


@torch.no_grad()
def extract_local_params_from_full_params(params, hidden_group, depth_group):
    """``[V, H]`` -> my hidden chunk -> flat -> my depth slice."""
    n, me = dist.get_world_size(hidden_group), dist.get_rank(hidden_group)
    h_l = params.shape[1] // n
    block = params[:, me * h_l:(me + 1) * h_l].contiguous().view(-1)
    nd, dz = dist.get_world_size(depth_group), dist.get_rank(depth_group)
    k = divide(block.numel(), nd)
    return block[dz * k:(dz + 1) * k].clone()


@torch.no_grad()
def default_init_method(weight, padding_idx=None):
    return torch.nn.init.normal_(weight)


class _EmbeddingRowsP2P(torch.autograd.Function):
    """Row lookup in a depth-sharded ``[V, H_l]`` table without gathering it."""

    @staticmethod
    def forward(ctx, ids, shard, group, rows_per_shard, row_elems, padding_idx):
        from ..parallel import fused

        flat = ids.reshape(-1)
        out = fused.embedding_fetch(group, flat, shard, rows_per_shard, row_elems)
        ctx.save_for_backward(flat)
        ctx.group, ctx.rows_per_shard, ctx.row_elems = group, rows_per_shard, row_elems
        ctx.shard_numel, ctx.shard_dtype, ctx.padding_idx = shard.numel(), shard.dtype, padding_idx
        return out.reshape(*ids.shape, row_elems)

    @staticmethod
    def backward(ctx, grad_out):
        from ..parallel import fused

        (flat,) = ctx.saved_tensors
        g = grad_out.reshape(-1, ctx.row_elems).to(torch.bfloat16)
        if ctx.padding_idx is not None:
            g = g.masked_fill((flat == ctx.padding_idx)[:, None], 0)
        gshard = fused.embedding_scatter_add(ctx.group, flat, g, ctx.rows_per_shard, ctx.row_elems, ctx.shard_numel)
        return None, gshard.to(ctx.shard_dtype), None, None, None, None


class Embedding(torch.nn.Module):
    """Drop-in ``nn.Embedding`` whose table is split along the embedding dimension over one tensor-parallel group
    (the outer group, or the inner one with ``transpose=True``) and flat-sharded over the depth group.  On GPUs
    with a depth group the needed rows are fetched from the owning ranks over peer memory instead of gathering
    the table (reference ``axonn/intra_layer/embedding.py:57-222``)."""

    def __init__(self, num_embeddings, embedding_dim, padding_idx=None, max_norm=None, norm_type=2.0,
                 scale_grad_by_freq=False, sparse=False, _weight=None, _freeze=False, *args,
                 transpose=False, init_method=None, expert_mode=False, dtype=None, **kwargs):
        assert _weight is None, "_weight argument is not supported."
        super().__init__()
        assert ax.is_initialized
        self.num_embeddings, self.embedding_dim = num_embeddings, embedding_dim
        if padding_idx is not None:
            if not -num_embeddings <= padding_idx < num_embeddings:
                raise ValueError("padding_idx must be within num_embeddings")
            if padding_idx < 0:
                padding_idx += num_embeddings
        self.padding_idx, self.max_norm, self.norm_type = padding_idx, max_norm, norm_type
        self.scale_grad_by_freq, self.sparse = scale_grad_by_freq, sparse
        ch = ax.comm_handle
        self.inner_group = ch.inner_intra_layer_parallel_group
        self.outer_group = ch.outer_intra_layer_parallel_group
        self.depth_group = ch.depth_intra_layer_parallel_group
        self.inner_group_size = dist.get_world_size(self.inner_group)
        self.outer_group_size = dist.get_world_size(self.outer_group)
        self.depth_group_size = dist.get_world_size(self.depth_group)
        self.transpose, self.expert_mode = transpose, expert_mode
        # The hidden dimension is split over one group.  In expert mode the table may
        # additionally be replicated over the other group (its ranks see the same
        # tokens and the same output gradient, so the replicas stay identical); in
        # easy mode the other group must have size one, as in the reference
        # (``embedding.py:110,123``).
        if not transpose:
            self.hidden_group, other = self.outer_group, self.inner_group_size
        else:
            self.hidden_group, other = self.inner_group, self.outer_group_size
        if other != 1 and not expert_mode:
            raise ValueError("easy-mode Embedding needs the non-hidden tensor-parallel group to have size 1")
        self.local_in_features = num_embeddings
        self.local_out_features = divide(embedding_dim, dist.get_world_size(self.hidden_group))
        self.in_features, self.out_features = num_embeddings, embedding_dim
        if init_method is None:
            init_method = default_init_method
        dtype = dtype or torch.get_default_dtype()
        full = torch.empty((num_embeddings, embedding_dim), device=ax.config.device, dtype=dtype)
        init_method(full)
        if padding_idx is not None:
            full[padding_idx].fill_(0)
        self.weight = torch.nn.Parameter(
            extract_local_params_from_full_params(full, self.hidden_group, self.depth_group),
            requires_grad=not _freeze)
        del full
        self.weight.is_tensor_parallel = True
        self.weight.needs_depth_parallel_gradient_sync = False
        self.weight.process_group_for_norm_reduction = ch.intra_layer_group
        self.weight.norm_reduction_replicas = other

    def get_output_feature_size(self):
        return self.local_out_features

    def _p2p_rows(self, x):
        """Peer-memory row fetch applies: depth > 1, whole rows per depth shard, plain lookup semantics."""
        import os

        if self.depth_group_size == 1 or not x.is_cuda or os.environ.get("AXONN_EMBEDDING_P2P", "1") == "0":
            return False
        if self.max_norm is not None or self.scale_grad_by_freq or self.sparse:
            return False
        if self.num_embeddings % self.depth_group_size:
            return False
        from ..parallel import fused

        return fused.embedding_p2p_usable(self.depth_group, self.weight,
                                          self.num_embeddings // self.depth_group_size, self.local_out_features)

    def forward(self, x):
        if self._p2p_rows(x):
            x = _EmbeddingRowsP2P.apply(x, self.weight, self.depth_group,
                                        self.num_embeddings // self.depth_group_size, self.local_out_features,
                                        self.padding_idx)
            if not self.expert_mode:
                x = Gather.apply(x, self.hidden_group)
            return x
        weight = ForwardGather_BackwardReduceScatter.apply(self.weight, self.depth_group).reshape(
            self.local_in_features, self.local_out_features)
        x = F.embedding(x, weight, self.padding_idx, self.max_norm, self.norm_type,
                        self.scale_grad_by_freq, self.sparse)
        if not self.expert_mode:
            x = Gather.apply(x, self.hidden_group)
        return x

    def _is_full_weight_matrix(self, w):
        return w.ndim == 2 and tuple(w.shape) == (self.num_embeddings, self.embedding_dim)

    def _is_sharded_weight_matrix(self, w):
        return w.ndim == 1 and w.size(0) == divide(
            self.local_in_features * self.local_out_features, self.depth_group_size)

    @torch.no_grad()
    def _load_from_state_dict(self, state_dict, prefix, *args, **kwargs):
        w = state_dict.get(prefix + "weight")
        if w is not None:
            if self._is_full_weight_matrix(w):
                state_dict[prefix + "weight"] = extract_local_params_from_full_params(
                    w, self.hidden_group, self.depth_group)
            elif not self._is_sharded_weight_matrix(w):
                raise ValueError("embedding weight is neither the full table nor this rank's shard")
        super()._load_from_state_dict(state_dict, prefix, *args, **kwargs)

    @torch.no_grad()
    def full_tensor(self, name, t=None):
        """Grid-independent ``[num_embeddings, embedding_dim]`` form of the table or of an optimizer state
        tensor laid out like it.  Collective over the depth and the hidden group."""
        t = self.weight.detach() if t is None else t
        w = _gather(t, 0, self.depth_group).reshape(self.local_in_features, self.local_out_features)
        return _gather(w, 1, self.hidden_group)

    @torch.no_grad()
    def shard_tensor(self, name, full):
        return extract_local_params_from_full_params(full, self.hidden_group, self.depth_group)
