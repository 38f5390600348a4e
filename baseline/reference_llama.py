"""Llama-style decoder built on the UNMODIFIED reference package (``axonn`` as
installed under ``baseline/_ref``) for the reference arm of ``bench.py --config llama8b``.

Parallelism comes from the reference's public API only: ``ax.init``,
``axonn.intra_layer.Linear(expert_mode=True)`` (depth-sharded weights: all-gather
before every use, reduce-scatter of the weight gradient), ``optimize_communication``
and ``sync_gradients``.  The rest is stock PyTorch (``nn.Embedding``, ``F.rms_norm``,
``F.scaled_dot_product_attention`` with grouped-query attention, ``F.silu``,
``torch.optim.AdamW``); nothing from ``axonn_b200`` is imported here.  The layer
structure follows what the reference's own Llama patch builds
(``axonn/models/transformers/modify_llama.py``: separate q/k/v/o and gate/up/down
projections, the output projections with ``transpose=True``).

Gradient pruning (keep the 10 % largest-magnitude entries of every gradient tensor)
is not in the reference snapshot; the baseline uses a plain PyTorch threshold
(``torch.kthvalue``) at the place the reference's pipeline engine offers for it
(after backward, before ``sync_gradients``).
"""

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F


def build(ref_axonn, cfg, device, prune_keep_fraction=0.1):
    """Return (model, train_step) where train_step(tokens, targets, micro_batch) -> loss tensor."""
    ax = ref_axonn.axonn
    il = ref_axonn.intra_layer
    Linear = il.Linear
    ch = ax.comm_handle
    inner, outer = ch.inner_intra_layer_parallel_group, ch.outer_intra_layer_parallel_group
    assert dist.get_world_size(inner) == 1 and dist.get_world_size(outer) == 1, \
        "this baseline covers the depth-only configuration (G_intra_r = G_intra_c = 1)"
    H, nh, nkv = cfg.hidden, cfg.n_heads, cfg.n_kv_heads
    D = H // nh

    def rope_tables(S):
        inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, D, 2, device=device, dtype=torch.float32) / D))
        ang = torch.outer(torch.arange(S, device=device, dtype=torch.float32), inv)
        return ang.cos()[None, :, None, :], ang.sin()[None, :, None, :]

    def rope(x, cos, sin):          # x [B, S, h, D], rotate-half form
        x1, x2 = x[..., : D // 2].float(), x[..., D // 2:].float()
        return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], -1).to(x.dtype)

    class Attention(nn.Module):
        def __init__(self):
            super().__init__()
            self.q = Linear(H, nh * D, bias=False, expert_mode=True)
            self.k = Linear(H, nkv * D, bias=False, expert_mode=True)
            self.v = Linear(H, nkv * D, bias=False, expert_mode=True)
            self.o = Linear(nh * D, H, bias=False, expert_mode=True, transpose=True)

        def forward(self, x, cos, sin):
            B, S, _ = x.shape
            q = rope(self.q(x).view(B, S, nh, D), cos, sin).transpose(1, 2)
            k = rope(self.k(x).view(B, S, nkv, D), cos, sin).transpose(1, 2)
            v = self.v(x).view(B, S, nkv, D).transpose(1, 2)
            o = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)
            return self.o(o.transpose(1, 2).reshape(B, S, nh * D))

    class Block(nn.Module):
        def __init__(self):
            super().__init__()
            self.n1 = nn.Parameter(torch.ones(H))
            self.n2 = nn.Parameter(torch.ones(H))
            self.attn = Attention()
            self.gate = Linear(H, cfg.ffn, bias=False, expert_mode=True)
            self.up = Linear(H, cfg.ffn, bias=False, expert_mode=True)
            self.down = Linear(cfg.ffn, H, bias=False, expert_mode=True, transpose=True)

        def forward(self, x, cos, sin):
            x = x + self.attn(F.rms_norm(x, (H,), self.n1.to(x.dtype), cfg.eps), cos, sin)
            h = F.rms_norm(x, (H,), self.n2.to(x.dtype), cfg.eps)
            return x + self.down(F.silu(self.gate(h)) * self.up(h))

    class Llama(nn.Module):
        def __init__(self):
            super().__init__()
            self.tok = nn.Embedding(cfg.vocab, H)
            nn.init.normal_(self.tok.weight, std=0.02)
            self.blocks = nn.ModuleList([Block() for _ in range(cfg.n_layers)])
            self.nf = nn.Parameter(torch.ones(H))
            self.head = Linear(H, cfg.vocab, bias=False, expert_mode=True)

        def forward(self, tokens, targets):
            cos, sin = rope_tables(tokens.shape[1])
            x = self.tok(tokens)
            if torch.is_autocast_enabled():
                x = x.to(torch.get_autocast_gpu_dtype())
            for b in self.blocks:
                x = b(x, cos, sin)
            logits = self.head(F.rms_norm(x, (H,), self.nf.to(x.dtype), cfg.eps))
            return F.cross_entropy(logits.float().view(-1, logits.shape[-1]), targets.reshape(-1))

    torch.manual_seed(1234)
    model = Llama().to(device)
    params = [p for p in model.parameters() if p.requires_grad]
    opt = torch.optim.AdamW(params, lr=1e-4, weight_decay=0.01, fused=True)

    @torch.no_grad()
    def prune(keep):
        for p in params:
            g = p.grad
            if g is None or g.numel() < 1024:
                continue
            n = g.numel()
            k = max(1, int(round(n * keep)))
            if k >= n:
                continue
            mag = g.detach().abs().reshape(-1)
            thr = mag.float().kthvalue(n - k + 1).values
            g.mul_((mag >= thr).to(g.dtype).view_as(g))

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
        if prune_keep_fraction is not None:
            prune(prune_keep_fraction)
        il.sync_gradients(model, mean=True, expert_mode=True)
        opt.step()
        opt.zero_grad(set_to_none=True)
        return total / n_micro

    return model, train_step
