"""Expert-parallel mixture-of-experts layer (top-k softmax router, SwiGLU experts).

Experts are partitioned over an expert-parallel group (by default the
data-parallel group: every data-parallel rank owns ``n_experts / G_data``
experts and routes its own tokens).  Tokens travel to the owners of their
experts and back with an all-to-all in each direction:

* on GPUs with peer memory the exchange is done by this package's dispatch and
  combine kernels (``csrc/moe.cu``): a token row is stored straight into the
  owning rank's expert buffer over NVLink while it is being gathered, and the
  expert outputs are pulled back, scaled by the gate and summed in one pass;
* otherwise ``all_to_all_single`` moves fixed-capacity buffers.

Fixed expert capacity keeps all shapes static (no host synchronisation):
``capacity = ceil(capacity_factor * tokens * top_k / n_experts)`` slots per
expert and source rank; assignments beyond it are dropped, as in
GShard/Switch routing.

The reference has no expert parallelism — its Mixtral patch only
tensor-parallelises every expert
(``axonn/models/transformers/modify_mixtral.py:86-97``); this layer is an
extension required for the Mixtral-style configuration.
"""

import math

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

from .. import axonn as ax
from .. import ops


class _AllToAll(torch.autograd.Function):
    """Equal-split all-to-all along dim 0; backward is the same exchange."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        if dist.get_world_size(group) == 1:
            return x
        x = x.contiguous()
        out = torch.empty_like(x)
        dist.all_to_all_single(out, x, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        if dist.get_world_size(ctx.group) == 1:
            return g, None
        g = g.contiguous()
        out = torch.empty_like(g)
        dist.all_to_all_single(out, g, group=ctx.group)
        return out, None


def route_top_k(logits, top_k, capacity):
    """Router decisions for ``logits`` [T, E].

    Returns (expert index [T, k], gate [T, k] renormalised over the chosen
    experts, slot [T, k] position inside the expert's capacity buffer, keep
    mask [T, k], auxiliary load-balancing loss)."""
    T, E = logits.shape
    probs = F.softmax(logits.float(), dim=-1)
    gate, idx = probs.topk(top_k, dim=-1)
    gate = gate / gate.sum(-1, keepdim=True)
    onehot = F.one_hot(idx.reshape(-1), E)                       # [T*k, E], token-major order
    slot = (onehot.cumsum(0) * onehot).sum(-1).reshape(T, top_k) - 1
    keep = slot < capacity
    # Switch-style balance loss: E * sum_e (fraction of assignments to e) * (mean router prob of e)
    frac = onehot.float().mean(0) * 1.0
    aux = E * (frac * probs.mean(0)).sum()
    return idx, gate, slot, keep, aux


class ExpertParallelMoE(nn.Module):
    """Mixture-of-experts feed-forward layer with whole experts placed on the ranks of ``ep_group`` (default: the
    data-parallel group): top-``top_k`` routing with a per-expert capacity of ``capacity_factor * tokens * top_k /
    n_experts`` rows, dispatch of the routed rows to the experts' ranks, SwiGLU experts as two batched GEMMs over
    all local experts, combine weighted by the gate values.  After a forward, ``last_aux_loss`` (load-balancing
    loss), ``last_drop_fraction``, ``last_assignments_per_expert`` and ``last_dropped_per_expert`` describe the
    routing (device tensors, no host synchronisation)."""

    def __init__(self, hidden, ffn, n_experts=8, top_k=2, capacity_factor=1.25, ep_group=None, dtype=None,
                 init_std=0.02, out_init_std=None):
        super().__init__()
        assert ax.is_initialized
        self.group = ep_group if ep_group is not None else ax.comm_handle.data_parallel_group
        self.ep = dist.get_world_size(self.group)
        self.ep_rank = dist.get_rank(self.group)
        assert n_experts % self.ep == 0, "n_experts must be divisible by the expert-parallel group size"
        self.hidden, self.ffn, self.n_experts, self.top_k = hidden, ffn, n_experts, top_k
        self.n_local = n_experts // self.ep
        self.capacity_factor = capacity_factor
        dev = ax.config.device
        self.router = nn.Parameter(torch.empty(n_experts, hidden, dtype=dtype, device=dev))
        nn.init.normal_(self.router, std=init_std)
        # materialise all experts with the shared RNG stream, keep mine (same weights for any ep size)
        w1 = torch.empty(n_experts, 2 * ffn, hidden, dtype=dtype, device=dev)
        w2 = torch.empty(n_experts, hidden, ffn, dtype=dtype, device=dev)
        nn.init.normal_(w1, std=init_std)
        nn.init.normal_(w2, std=out_init_std or init_std)
        lo, hi = self.ep_rank * self.n_local, (self.ep_rank + 1) * self.n_local
        self.w1 = nn.Parameter(w1[lo:hi].clone())   # [gate|up] interleaved in blocks of 8 rows (ops.swiglu layout)
        self.w2 = nn.Parameter(w2[lo:hi].clone())
        del w1, w2
        for p in (self.w1, self.w2):
            p.is_expert_parallel = self.ep > 1
        self.last_aux_loss = None
        self.last_drop_fraction = None
        self.last_assignments_per_expert = None
        self.last_dropped_per_expert = None

    @torch.no_grad()
    def full_tensor(self, name, t=None):
        """All experts' ``w1`` / ``w2`` (``[n_experts, ...]``; or an optimizer state tensor laid out like them),
        gathered over the expert-parallel group; the router is replicated and returned as it is."""
        t = getattr(self, name).detach() if t is None else t
        if name == "router" or self.ep == 1:
            return t
        out = torch.empty((self.n_experts,) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
        dist.all_gather_into_tensor(out, t.contiguous(), group=self.group)
        return out

    @torch.no_grad()
    def shard_tensor(self, name, full):
        if name == "router" or self.ep == 1:
            return full
        return full[self.ep_rank * self.n_local:(self.ep_rank + 1) * self.n_local].clone()

    def _load_from_state_dict(self, state_dict, prefix, *args, **kwargs):
        """Accept ``w1`` / ``w2`` holding all experts (a checkpoint of another grid) as well as the local ones."""
        if self.ep > 1:
            for name in ("w1", "w2"):
                v = state_dict.get(prefix + name)
                if v is not None and v.shape[0] == self.n_experts:
                    state_dict[prefix + name] = self.shard_tensor(name, v)
        super()._load_from_state_dict(state_dict, prefix, *args, **kwargs)

    def capacity(self, tokens):
        c = math.ceil(self.capacity_factor * tokens * self.top_k / self.n_experts)
        return max(8, (c + 7) // 8 * 8)

    def _experts(self, x, seg=None, seg_rows=0):
        """x: [n_local, rows, H] -> [n_local, rows, H].  One launch per GEMM over the tiles of all local experts
        (capacity buffers make the shapes uniform).  ``seg`` (int32 [n_local, rows / seg_rows]): how many rows of
        each ``seg_rows``-row capacity segment hold tokens - the others are zero, and the GEMMs skip the tiles
        (weight gradient: the K blocks) that contain none."""
        h = ops.swiglu(ops.linear_batched(x, self.w1, seg, seg_rows))
        return ops.linear_batched(h, self.w2, seg, seg_rows)

    def forward(self, x):
        shape = x.shape
        x2 = x.reshape(-1, self.hidden)
        T = x2.shape[0]
        C = self.capacity(T)
        E, k = self.n_experts, self.top_k
        logits = ops.linear(x2, self.router)
        idx, gate, slot, keep, aux = route_top_k(logits, k, C)
        self.last_aux_loss = aux
        self.last_drop_fraction = 1.0 - keep.float().mean().detach()
        # routing statistics of this rank's tokens (device tensors, no host synchronisation): assignments per
        # expert before the capacity cut, and how many of them were dropped per expert
        with torch.no_grad():
            flat_idx = idx.reshape(-1)
            ones = torch.ones(flat_idx.shape, dtype=torch.float32, device=flat_idx.device)
            zeros = torch.zeros(E, dtype=torch.float32, device=flat_idx.device)
            self.last_assignments_per_expert = zeros.index_add(0, flat_idx, ones)
            self.last_dropped_per_expert = zeros.index_add(0, flat_idx, (~keep).reshape(-1).float())
        dest = (idx * C + slot.clamp(max=C - 1)).reshape(-1)           # row in the [E*C, H] send buffer
        keep_f = keep.reshape(-1)
        from . import moe_kernels

        if moe_kernels.usable(self.group, x2):
            y = moe_kernels.dispatch_experts_combine(self, x2, dest, keep_f, gate.reshape(-1), C)
            return y.reshape(shape)
        src_tok = torch.arange(T, device=x.device).repeat_interleave(k)
        send = x2.new_zeros(E * C, self.hidden)
        send = send.index_copy(0, dest[keep_f], x2.index_select(0, src_tok[keep_f]))
        # [E, C, H] = [ep, n_local, C, H]: chunk j goes to rank j; received [ep(src), n_local, C, H]
        recv = _AllToAll.apply(send.reshape(self.ep, self.n_local * C, self.hidden), self.group)
        recv = recv.reshape(self.ep, self.n_local, C, self.hidden).transpose(0, 1)
        out = self._experts(recv.reshape(self.n_local, self.ep * C, self.hidden))
        out = out.reshape(self.n_local, self.ep, C, self.hidden).transpose(0, 1)
        back = _AllToAll.apply(out.reshape(self.ep, self.n_local * C, self.hidden), self.group)
        back = back.reshape(E * C, self.hidden)
        picked = back.index_select(0, dest) * (gate.reshape(-1) * keep_f).to(back.dtype)[:, None]
        y = picked.reshape(T, k, self.hidden).sum(1)
        return y.reshape(shape)
