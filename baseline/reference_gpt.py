"""GPT-style decoder built on the UNMODIFIED reference package (``axonn`` as
installed under ``baseline/_ref``) for the reference arm of ``bench.py``.

Only the reference's public API is used for parallelism: ``ax.init``,
``axonn.intra_layer.Linear(expert_mode=True)``, ``Drop``,
``optimize_communication`` and ``sync_gradients``.  Everything else is stock
PyTorch (``nn.Embedding``, ``F.scaled_dot_product_attention``, ``F.gelu``,
``torch.optim.AdamW``); nothing from ``axonn_b200`` is imported here.  The
reference ships no runnable GPT of its own (its ``external/models`` needs a
Megatron fork), so the architecture is restated with the same layout rules as
the product's model: hidden split over the column group between blocks, heads
over the row group, vocabulary over the row group.
"""


import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F


def build(ref_axonn, cfg, device, bf16_params=False):
    """Return (model, train_step) where train_step(tokens, targets, n_micro) -> loss tensor.

    ``bf16_params=True`` is a diagnostic variant: the whole model is cast to bf16 (no fp32 master weights, no
    weight cast per GEMM, bf16 depth all-gathers), which is not the mixed-precision recipe the reference's
    ``AsyncLinear`` is written for but shows how much of a speed difference is recipe and how much kernels."""
    ax = ref_axonn.axonn
    il = ref_axonn.intra_layer
    Linear, Drop = il.Linear, il.Drop
    ch = ax.comm_handle
    inner, outer = ch.inner_intra_layer_parallel_group, ch.outer_intra_layer_parallel_group
    c, r = dist.get_world_size(inner), dist.get_world_size(outer)

    class _AllReduceSum(torch.autograd.Function):
        """Sum over a group in forward and in backward (statistics of sharded rows)."""

        @staticmethod
        def forward(ctx, x, group):
            ctx.group = group
            x = x.clone()
            dist.all_reduce(x, group=group)
            return x

        @staticmethod
        def backward(ctx, g):
            g = g.clone()
            dist.all_reduce(g, group=ctx.group)
            return g, None

    class ShardedLayerNorm(nn.Module):
        def __init__(self, hidden, eps=1e-5):
            super().__init__()
            self.hidden, self.eps = hidden, eps
            self.weight = nn.Parameter(torch.ones(hidden // c))
            self.bias = nn.Parameter(torch.zeros(hidden // c))

        def forward(self, x):
            if c == 1:
                return F.layer_norm(x, (self.hidden,), self.weight, self.bias, self.eps)
            xf = x.float()
            stats = torch.stack([xf.sum(-1), (xf * xf).sum(-1)], -1)
            stats = _AllReduceSum.apply(stats, inner)
            mean = stats[..., 0:1] / self.hidden
            var = stats[..., 1:2] / self.hidden - mean * mean
            y = (xf - mean) * torch.rsqrt(var + self.eps)
            return (y * self.weight.float() + self.bias.float()).to(x.dtype)

    class Attention(nn.Module):
        def __init__(self):
            super().__init__()
            self.hl, self.D = cfg.n_heads // r, cfg.hidden // cfg.n_heads
            self.qkv = Linear(cfg.hidden, 3 * cfg.hidden, expert_mode=True)
            self.proj = Linear(cfg.hidden, cfg.hidden, expert_mode=True, transpose=True)

        def forward(self, x):
            B, S, _ = x.shape
            qkv = self.qkv(x).view(B, S, self.hl, 3, self.D)
            q, k, v = (qkv[:, :, :, i].transpose(1, 2) for i in range(3))
            o = F.scaled_dot_product_attention(q, k, v, is_causal=True)
            return self.proj(o.transpose(1, 2).reshape(B, S, self.hl * self.D))

    class Block(nn.Module):
        def __init__(self):
            super().__init__()
            self.n1, self.n2 = ShardedLayerNorm(cfg.hidden), ShardedLayerNorm(cfg.hidden)
            self.attn = Attention()
            self.fc1 = Linear(cfg.hidden, cfg.ffn, expert_mode=True)
            self.fc2 = Linear(cfg.ffn, cfg.hidden, expert_mode=True, transpose=True)

        def forward(self, x):
            x = x + self.attn(self.n1(x))
            return x + self.fc2(F.gelu(self.fc1(self.n2(x)), approximate="tanh"))

    class VocabParallelCE(torch.autograd.Function):
        @staticmethod
        def forward(ctx, logits, targets):
            V = logits.shape[-1]
            z = logits.float().reshape(-1, V)
            t = targets.reshape(-1)
            start = dist.get_rank(outer) * V
            m = z.max(-1).values
            dist.all_reduce(m, op=dist.ReduceOp.MAX, group=outer)
            e = (z - m[:, None]).exp()
            s = e.sum(-1)
            loc = t - start
            inside = (loc >= 0) & (loc < V)
            tl = torch.where(inside, z.gather(1, loc.clamp(0, V - 1)[:, None])[:, 0], torch.zeros_like(m))
            st = torch.stack([s, tl])
            dist.all_reduce(st, group=outer)
            s, tl = st[0], st[1]
            loss = (m + s.log() - tl).mean()
            p = e / s[:, None]
            p[inside, loc[inside]] -= 1.0
            ctx.save_for_backward(p)
            ctx.shape, ctx.dtype = logits.shape, logits.dtype
            return loss

        @staticmethod
        def backward(ctx, g):
            (p,) = ctx.saved_tensors
            return (p * (g / p.shape[0])).to(ctx.dtype).reshape(ctx.shape), None

    class GPT(nn.Module):
        def __init__(self):
            super().__init__()
            self.tok = nn.Embedding(cfg.vocab, cfg.hidden)
            self.pos = nn.Embedding(cfg.seq_len, cfg.hidden)
            nn.init.normal_(self.tok.weight, std=0.02)
            nn.init.normal_(self.pos.weight, std=0.02)
            self.blocks = nn.ModuleList([Block() for _ in range(cfg.n_layers)])
            self.nf = ShardedLayerNorm(cfg.hidden)
            self.head = Linear(cfg.hidden, cfg.vocab, bias=False, expert_mode=True)

        def forward(self, tokens, targets):
            S = tokens.shape[1]
            x = self.tok(tokens) + self.pos(torch.arange(S, device=tokens.device))[None]
            x = Drop.apply(x, inner)  # hidden split over the column group
            for b in self.blocks:
                x = b(x)
            logits = self.head(self.nf(x))
            if r == 1:
                return F.cross_entropy(logits.float().view(-1, logits.shape[-1]), targets.reshape(-1))
            return VocabParallelCE.apply(logits, targets)

    torch.manual_seed(1234)
    model = GPT().to(device)
    if bf16_params:
        model = model.to(torch.bfloat16)
    # parameters that are replicated inside the tensor-parallel group are ordinary
    # (non-"tensor parallel") parameters for the reference's sync_gradients
    opt = torch.optim.AdamW(model.parameters(), lr=1e-4, weight_decay=0.01, fused=True)

    def train_step(tokens, targets, micro_batch):
        B = tokens.shape[0]
        n_micro = max(1, B // micro_batch)
        total = None
        for i in range(n_micro):
            x, y = tokens[i * micro_batch:(i + 1) * micro_batch], targets[i * micro_batch:(i + 1) * micro_batch]
            with il.optimize_communication(overlap_all_reduce=True, overlap_reduce_scatter=True,
                                           overlap_all_gather=True, model_object_for_overlapping_allgathers=model):
                with torch.autocast("cuda", dtype=torch.bfloat16):
                    loss = model(x, y)
                (loss / n_micro).backward()
            total = loss.detach() if total is None else total + loss.detach()
        il.sync_gradients(model, mean=True, expert_mode=True)
        opt.step()
        opt.zero_grad(set_to_none=True)
        return total / n_micro

    return model, train_step
