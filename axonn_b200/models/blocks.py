"""Tensor-parallel transformer building blocks (expert-mode layout).

Activation layout between blocks: ``[batch_local, seq, hidden / G_c]`` — the
hidden dimension is split over the column ("inner") group, the batch over the
depth and data groups, and everything is replicated over the row group.  A
non-transposed ``Linear`` consumes that layout and produces features split
over the row group; a transposed ``Linear`` maps back.  Attention heads are
therefore split over the row group, and normalisation layers reduce their row
statistics over the column group.

These modules replace the HF monkey patches of the reference
(``axonn/models/transformers/modify_*.py``) and Megatron's ``ParallelTransformer``
used by ``external/models/nvidia_transformer.py``.
"""

import math

import torch
import torch.distributed as dist
import torch.nn as nn

from .. import axonn as ax
from .. import ops
from ..intra_layer import Gather, Linear
from ..intra_layer.communication import _drop, _gather
from ..utils import divide


def _groups():
    ch = ax.comm_handle
    return ch.inner_intra_layer_parallel_group, ch.outer_intra_layer_parallel_group


def _tag_sharded(param, shard_group):
    """Bookkeeping for a parameter sharded over ``shard_group`` and replicated over depth."""
    param.is_tensor_parallel = True
    param.needs_depth_parallel_gradient_sync = True
    param.process_group_for_norm_reduction = shard_group
    return param


class TPNorm(nn.Module):
    """LayerNorm / RMSNorm whose hidden dimension is split over the column group."""

    def __init__(self, hidden, eps=1e-5, rms=False, dtype=None):
        super().__init__()
        inner, _ = _groups()
        self.group = inner if dist.get_world_size(inner) > 1 else None
        self.local = divide(hidden, dist.get_world_size(inner))
        dev = ax.config.device
        self.weight = nn.Parameter(torch.ones(self.local, dtype=dtype, device=dev))
        self.bias = None if rms else nn.Parameter(torch.zeros(self.local, dtype=dtype, device=dev))
        self.eps, self.rms = eps, rms
        for p in self.parameters():
            _tag_sharded(p, inner)

    def forward(self, x):
        if self.rms:
            return ops.rms_norm(x, self.weight, self.eps, self.group)
        return ops.layer_norm(x, self.weight, self.bias, self.eps, self.group)

    @torch.no_grad()
    def full_tensor(self, name, t=None):
        """The whole ``[hidden]`` vector of ``weight`` / ``bias`` (or of an optimizer state tensor laid out like
        it); collective over the column group."""
        t = getattr(self, name).detach() if t is None else t
        return t if self.group is None else _gather(t, 0, self.group)

    @torch.no_grad()
    def shard_tensor(self, name, full):
        return full if self.group is None else _drop(full, 0, self.group).clone()

    def _load_from_state_dict(self, state_dict, prefix, *args, **kwargs):
        """Accept the full ``[hidden]`` vectors (a checkpoint of another grid) as well as this rank's slices."""
        if self.group is not None:
            for name in ("weight", "bias"):
                v = state_dict.get(prefix + name)
                if v is not None and v.numel() == self.local * dist.get_world_size(self.group):
                    state_dict[prefix + name] = self.shard_tensor(name, v)
        super()._load_from_state_dict(state_dict, prefix, *args, **kwargs)

    def add_norm(self, x, delta):
        """``h = x + delta`` and ``norm(h)`` in one kernel (the residual add fused into the normalisation);
        returns ``(h, norm(h))``."""
        if self.rms:
            return ops.add_rms_norm(x, delta, self.weight, self.eps, self.group)
        return ops.add_layer_norm(x, delta, self.weight, self.bias, self.eps, self.group)


class ParallelAttention(nn.Module):
    """Causal self-attention; KV groups (a KV head with its query heads) are split
    over the row group.

    The fused projection's output features are ordered group by group:
    ``[q heads of group 0 | k_0 | v_0 | q heads of group 1 | k_1 | v_1 | ...]``, so a
    contiguous slice of the rows of the weight holds whole groups and the model
    is the same function for every tensor-parallel degree."""

    def __init__(self, hidden, n_heads, n_kv_heads=None, bias=True, rope_theta=None, max_seq=4096, dtype=None,
                 init_std=0.02, out_init_std=None):
        super().__init__()
        _, outer = _groups()
        r = dist.get_world_size(outer)
        n_kv_heads = n_kv_heads or n_heads
        self.head_dim = divide(hidden, n_heads)
        self.q_per_kv = divide(n_heads, n_kv_heads)
        self.groups_l = divide(n_kv_heads, r)
        self.rope_theta, self.max_seq = rope_theta, max_seq
        self.sequence_group = None     # set by parallel.sequence.enable_sequence_parallel
        qkv_out = (n_heads + 2 * n_kv_heads) * self.head_dim
        self.qkv = Linear(hidden, qkv_out, bias=bias, expert_mode=True, dtype=dtype,
                          init_method=lambda w: nn.init.normal_(w, std=init_std))
        self.proj = Linear(n_heads * self.head_dim, hidden, bias=bias, expert_mode=True, transpose=True,
                           init_method=lambda w: nn.init.normal_(w, std=out_init_std or init_std), dtype=dtype)

    def forward(self, x):
        B, S, _ = x.shape
        D, G, qpk = self.head_dim, self.groups_l, self.q_per_kv
        qkv = self.qkv(x).view(B, S, G, qpk + 2, D)
        if self.sequence_group is not None:
            # x holds a slice of every sequence: trade it for whole sequences of a share of the heads, attend,
            # trade back (rotary embedding in between, on whole sequences)
            from ..parallel.sequence import ulysses_attention_packed

            o = ulysses_attention_packed(qkv, self.sequence_group, self._rope if self.rope_theta is not None else None)
        else:
            if self.rope_theta is not None:
                qkv = self._rope(qkv)
            o = ops.flash_attention_packed(qkv, causal=True)  # [B, S, G * qpk, D]
        return self.proj(o.reshape(B, S, G * qpk * D))

    def _rope(self, qkv):
        """Rotary embedding of the query heads and the key head of every group of ``[B, S, groups, q_per_kv + 2, D]``
        (positions 0 .. S-1)."""
        S, qpk, D = qkv.shape[1], self.q_per_kv, self.head_dim
        table = ops.rope_table(max(S, self.max_seq), D, self.rope_theta, qkv.device)
        if qkv.is_cuda:
            ops.apply_rope(qkv[:, :, :, :qpk + 1], table)  # in place
            return qkv
        return torch.cat([ops.apply_rope(qkv[:, :, :, :qpk + 1], table), qkv[:, :, :, qpk + 1:]], 3)


class ParallelMLP(nn.Module):
    """``fc2(act(fc1(x)))`` with GELU, or SwiGLU with a fused gate|up projection."""

    def __init__(self, hidden, ffn, activation="gelu", bias=True, dtype=None, init_std=0.02, out_init_std=None):
        super().__init__()
        self.activation = activation
        mult = 2 if activation == "swiglu" else 1
        _, outer = _groups()
        self.ffn_l = divide(ffn, dist.get_world_size(outer))
        # SwiGLU: gate and up rows are interleaved in blocks of 8 (see ops.swiglu), so any
        # contiguous row slice of the fused weight is self-contained
        self.fc1 = Linear(hidden, mult * ffn, bias=bias, expert_mode=True, dtype=dtype,
                          init_method=lambda w: nn.init.normal_(w, std=init_std))
        self.fc2 = Linear(ffn, hidden, bias=bias, expert_mode=True, transpose=True, dtype=dtype,
                          init_method=lambda w: nn.init.normal_(w, std=out_init_std or init_std))

    def forward(self, x):
        if self.activation == "swiglu":
            return self.fc2(ops.swiglu(self.fc1(x)))
        return self.fc2(self.fc1(x, activation="gelu"))


class TransformerBlock(nn.Module):
    """Pre-norm block: ``x + attn(norm1(x))`` then ``+ mlp(norm2(.))``, LayerNorm or RMSNorm, GELU or SwiGLU."""

    def __init__(self, hidden, n_heads, ffn, n_kv_heads=None, activation="gelu", rms=False, bias=True,
                 rope_theta=None, max_seq=4096, eps=1e-5, dtype=None, n_layers=1):
        super().__init__()
        out_std = 0.02 / math.sqrt(2 * n_layers)
        self.norm1 = TPNorm(hidden, eps, rms, dtype)
        self.attn = ParallelAttention(hidden, n_heads, n_kv_heads, bias, rope_theta, max_seq, dtype,
                                      out_init_std=out_std)
        self.norm2 = TPNorm(hidden, eps, rms, dtype)
        self.mlp = self._make_mlp(hidden, ffn, activation, bias, dtype, out_std)

    def _make_mlp(self, hidden, ffn, activation, bias, dtype, out_std):
        return ParallelMLP(hidden, ffn, activation, bias, dtype, out_init_std=out_std)

    def forward_deferred(self, x, delta=None):
        """The block with its residual adds fused into the normalisation kernels.  ``delta`` is the output of
        the previous block's MLP that has not been added to the residual stream ``x`` yet; returns
        ``(residual stream, this block's MLP output)`` - the caller (the next block, or the model's final norm)
        performs the last add inside its own norm kernel."""
        if delta is None:
            y = self.norm1(x)
        else:
            x, y = self.norm1.add_norm(x, delta)
        a = self.attn(y)
        x, y = self.norm2.add_norm(x, a)
        return x, self.mlp(y)

    def forward(self, x):
        x, m = self.forward_deferred(x)
        return x + m


class ParallelLMHead(nn.Module):
    """Final projection to a vocabulary split over the whole row x column grid + parallel cross-entropy.

    With a column group of one the projection is the ordinary non-transposed layer (vocabulary over the row
    group).  With ``G_intra_c > 1`` that layer would all-reduce the ``[tokens, vocab / r]`` logits over the
    column group - by far the largest tensor of the model.  Instead the hidden dimension of the input is
    all-gathered over the column group (``tokens x hidden``, small) and the vocabulary is split over all
    ``r * c`` ranks (a per-layer ``tensor_parallel_dims=(r*c, 1, d)``): the logits need no reduction at all,
    the input gradient is all-reduced over the ``r * c`` ranks, and the gather's backward keeps this rank's
    hidden chunk of that (already complete) gradient."""

    def __init__(self, hidden, vocab, dtype=None):
        super().__init__()
        inner, outer = _groups()
        r, c = dist.get_world_size(outer), dist.get_world_size(inner)
        self.gather_group = None
        dims = None
        if c > 1 and vocab % (r * c) == 0:
            self.gather_group = inner
            dims = (r * c, 1, ax.config.G_intra_d)
        self.proj = Linear(hidden, vocab, bias=False, expert_mode=True, dtype=dtype,
                           init_method=lambda w: nn.init.normal_(w, std=0.02), tensor_parallel_dims=dims)
        vocab_group = self.proj.outer_group
        self.group = vocab_group if dist.get_world_size(vocab_group) > 1 else None

    def forward(self, x, targets=None):
        if self.gather_group is not None:
            x = Gather.apply(x, self.gather_group, -1)
        logits = self.proj(x)
        if targets is None:
            return logits
        return ops.cross_entropy(logits, targets, group=self.group)


def count_parameters(module, local=False):
    """Global (or local) parameter count of a tensor-parallel module."""
    total = 0
    for p in module.parameters():
        n = p.numel()
        if not local and getattr(p, "is_tensor_parallel", False):
            g = getattr(p, "process_group_for_norm_reduction", None)
            if g is not None:
                n *= dist.get_world_size(g)
        total += n
    return total
