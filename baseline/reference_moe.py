"""Plain-PyTorch baseline of the expert-parallel Mixtral-style configuration
(``bench.py --config mixtral --impl reference``).

The reference has no expert parallelism (its Mixtral patch only tensor-parallelises every expert,
``axonn/models/transformers/modify_mixtral.py:86-97``), so there is no reference code to run for this
configuration.  The baseline is the same algorithm written with stock PyTorch and NCCL only (nothing from
``axonn_b200`` is imported): top-2 softmax router with a Switch-style balance loss, fixed expert capacity,
``all_to_all_single`` dispatch and combine, one cuBLAS GEMM pair per local expert, SDPA attention with
grouped-query heads, ``F.rms_norm``, bf16 autocast over fp32 parameters, fused ``torch.optim.AdamW`` and one
flat NCCL all-reduce for the gradients of the replicated (non-expert) parameters.
"""

import math

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F


class _AllToAll(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        x = x.contiguous()
        out = torch.empty_like(x)
        dist.all_to_all_single(out, x)
        return out

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        out = torch.empty_like(g)
        dist.all_to_all_single(out, g)
        return out


def build(cfg, device, world, rank):
    """Return (model, train_step) where train_step(tokens, targets, micro_batch) -> loss tensor."""
    H, nh, nkv, E, k = cfg.hidden, cfg.n_heads, cfg.n_kv_heads, cfg.n_experts, cfg.top_k
    D = H // nh
    n_local = E // world

    def rope_tables(S):
        inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, D, 2, device=device, dtype=torch.float32) / D))
        ang = torch.outer(torch.arange(S, device=device, dtype=torch.float32), inv)
        return ang.cos()[None, :, None, :], ang.sin()[None, :, None, :]

    def rope(x, cos, sin):
        x1, x2 = x[..., : D // 2].float(), x[..., D // 2:].float()
        return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], -1).to(x.dtype)

    class Attention(nn.Module):
        def __init__(self):
            super().__init__()
            self.qkv = nn.Linear(H, (nh + 2 * nkv) * D, bias=False)
            self.o = nn.Linear(nh * D, H, bias=False)

        def forward(self, x, cos, sin):
            B, S, _ = x.shape
            q, kk, v = self.qkv(x).split([nh * D, nkv * D, nkv * D], -1)
            q = rope(q.view(B, S, nh, D), cos, sin).transpose(1, 2)
            kk = rope(kk.view(B, S, nkv, D), cos, sin).transpose(1, 2)
            v = v.view(B, S, nkv, D).transpose(1, 2)
            o = F.scaled_dot_product_attention(q, kk, v, is_causal=True, enable_gqa=True)
            return self.o(o.transpose(1, 2).reshape(B, S, nh * D))

    class MoE(nn.Module):
        def __init__(self):
            super().__init__()
            self.router = nn.Linear(H, E, bias=False)
            self.w_gate = nn.Parameter(torch.empty(n_local, cfg.ffn, H))
            self.w_up = nn.Parameter(torch.empty(n_local, cfg.ffn, H))
            self.w_down = nn.Parameter(torch.empty(n_local, H, cfg.ffn))
            for p in (self.w_gate, self.w_up, self.w_down):
                nn.init.normal_(p, std=0.02)
                p.is_expert = True
            self.aux = None

        def forward(self, x):
            shape = x.shape
            x2 = x.reshape(-1, H)
            T = x2.shape[0]
            C = max(8, (math.ceil(cfg.capacity_factor * T * k / E) + 7) // 8 * 8)
            probs = F.softmax(self.router(x2).float(), -1)
            gate, idx = probs.topk(k, -1)
            gate = gate / gate.sum(-1, keepdim=True)
            onehot = F.one_hot(idx.reshape(-1), E)
            slot = (onehot.cumsum(0) * onehot).sum(-1).reshape(T, k) - 1
            keep = (slot < C).reshape(-1)
            self.aux = E * (onehot.float().mean(0) * probs.mean(0)).sum()
            dest = (idx * C + slot.clamp(max=C - 1)).reshape(-1)
            src_tok = torch.arange(T, device=x.device).repeat_interleave(k)
            send = x2.new_zeros(E * C, H).index_copy(0, dest[keep], x2.index_select(0, src_tok[keep]))
            recv = _AllToAll.apply(send.reshape(world, n_local * C, H)) if world > 1 else send.reshape(world, n_local * C, H)
            recv = recv.reshape(world, n_local, C, H).transpose(0, 1).reshape(n_local, world * C, H)
            outs = []
            for e in range(n_local):
                h = F.silu(F.linear(recv[e], self.w_gate[e].to(recv.dtype))) * F.linear(recv[e], self.w_up[e].to(recv.dtype))
                outs.append(F.linear(h, self.w_down[e].to(recv.dtype)))
            out = torch.stack(outs, 0).reshape(n_local, world, C, H).transpose(0, 1).reshape(world, n_local * C, H)
            back = (_AllToAll.apply(out) if world > 1 else out).reshape(E * C, H)
            picked = back.index_select(0, dest) * (gate.reshape(-1) * keep).to(back.dtype)[:, None]
            return picked.reshape(T, k, H).sum(1).reshape(shape)

    class Block(nn.Module):
        def __init__(self):
            super().__init__()
            self.n1, self.n2 = nn.Parameter(torch.ones(H)), nn.Parameter(torch.ones(H))
            self.attn, self.moe = Attention(), MoE()

        def forward(self, x, cos, sin):
            x = x + self.attn(F.rms_norm(x, (H,), self.n1.to(x.dtype), cfg.eps), cos, sin)
            return x + self.moe(F.rms_norm(x, (H,), self.n2.to(x.dtype), cfg.eps))

    class Model(nn.Module):
        def __init__(self):
            super().__init__()
            self.tok = nn.Embedding(cfg.vocab, H)
            self.blocks = nn.ModuleList([Block() for _ in range(cfg.n_layers)])
            self.nf = nn.Parameter(torch.ones(H))
            self.head = nn.Linear(H, cfg.vocab, bias=False)

        def forward(self, tokens, targets):
            cos, sin = rope_tables(tokens.shape[1])
            x = self.tok(tokens).to(torch.bfloat16)
            for b in self.blocks:
                x = b(x, cos, sin)
            logits = self.head(F.rms_norm(x, (H,), self.nf.to(x.dtype), cfg.eps))
            loss = F.cross_entropy(logits.float().view(-1, logits.shape[-1]), targets.reshape(-1))
            aux = sum(b.moe.aux for b in self.blocks) / len(self.blocks)
            return loss + cfg.aux_loss_coef * aux

    torch.manual_seed(1234 + rank)      # experts differ per rank; replicated parameters are broadcast below
    model = Model().to(device)
    shared = [p for p in model.parameters() if not getattr(p, "is_expert", False)]
    if world > 1:
        for p in shared:
            dist.broadcast(p.data, src=0)
    opt = torch.optim.AdamW(model.parameters(), lr=1e-4, weight_decay=0.01, fused=True)

    def train_step(tokens, targets, micro_batch):
        B = tokens.shape[0]
        n_micro = max(1, B // micro_batch)
        total = None
        for i in range(n_micro):
            x, y = tokens[i * micro_batch:(i + 1) * micro_batch], targets[i * micro_batch:(i + 1) * micro_batch]
            with torch.autocast("cuda", dtype=torch.bfloat16):
                loss = model(x, y)
            (loss / n_micro).backward()
            total = loss.detach() if total is None else total + loss.detach()
        if world > 1:
            grads = [p.grad for p in shared if p.grad is not None]
            flat = torch._utils._flatten_dense_tensors(grads)
            dist.all_reduce(flat)
            flat.div_(world)
            for g, new in zip(grads, torch._utils._unflatten_dense_tensors(flat, grads)):
                g.copy_(new)
            for p in model.parameters():
                if getattr(p, "is_expert", False) and p.grad is not None:
                    p.grad.div_(world)
        opt.step()
        opt.zero_grad(set_to_none=True)
        return total / n_micro

    return model, train_step
