"""Mixtral-style sparse mixture-of-experts decoder: RMSNorm, rotary embeddings,
grouped-query attention and, in place of the dense MLP, ``n_experts`` SwiGLU
experts with a top-2 softmax router and a load-balancing auxiliary loss.
``MixtralConfig.mixtral_16l()`` is the benchmark configuration (16 layers,
d_model 4096, 32 / 8 heads, 8 experts of FFN 14336, vocabulary 32000, sequence
4096) with experts partitioned over the data-parallel group.

The reference only tensor-parallelises Mixtral's experts through an HF patch
(``axonn/models/transformers/modify_mixtral.py``); this is a native model with
expert parallelism.
"""

from dataclasses import dataclass

import torch
import torch.nn as nn
from torch.utils.checkpoint import checkpoint

from ..intra_layer import Embedding
from ..parallel.moe import ExpertParallelMoE
from .blocks import ParallelLMHead, TPNorm, TransformerBlock, count_parameters


@dataclass
class MixtralConfig:
    """Shape of a Mixtral-style model; ``mixtral_16l()`` is the benchmark configuration, ``tiny()`` the test one."""

    n_layers: int = 16
    hidden: int = 4096
    n_heads: int = 32
    n_kv_heads: int = 8
    ffn: int = 14336
    n_experts: int = 8
    top_k: int = 2
    vocab: int = 32000
    seq_len: int = 4096
    rope_theta: float = 1e6
    eps: float = 1e-5
    aux_loss_coef: float = 0.02
    capacity_factor: float = 1.25
    activation_checkpointing: bool = False

    @staticmethod
    def mixtral_16l(**kw):
        return MixtralConfig(**kw)

    @staticmethod
    def tiny(**kw):
        return MixtralConfig(n_layers=2, hidden=128, n_heads=4, n_kv_heads=2, ffn=256, n_experts=4, vocab=512,
                             seq_len=64, **kw)

    def flops_per_token(self):
        """Active-parameter FLOPs per token (top_k experts), forward + backward."""
        h, L = self.hidden, self.n_layers
        hd = h // self.n_heads
        per_layer = 2 * h * h + 2 * h * self.n_kv_heads * hd + self.top_k * 3 * h * self.ffn + h * self.n_experts
        return 6 * (L * per_layer + h * self.vocab) + 6 * L * self.seq_len * h


class MoEBlock(TransformerBlock):
    def __init__(self, cfg: MixtralConfig, dtype):
        self._cfg = cfg
        super().__init__(cfg.hidden, cfg.n_heads, cfg.ffn, n_kv_heads=cfg.n_kv_heads, activation="swiglu", rms=True,
                         bias=False, rope_theta=cfg.rope_theta, max_seq=cfg.seq_len, eps=cfg.eps, dtype=dtype,
                         n_layers=cfg.n_layers)

    def _make_mlp(self, hidden, ffn, activation, bias, dtype, out_std):
        c = self._cfg
        return ExpertParallelMoE(hidden, ffn, c.n_experts, c.top_k, c.capacity_factor, dtype=dtype,
                                 out_init_std=out_std)


class Mixtral(nn.Module):
    """Decoder-only transformer with RMSNorm, rotary grouped-query attention and an ``ExpertParallelMoE``
    feed-forward in every block; ``forward(tokens, targets)`` returns the loss including the routers' auxiliary
    loss, ``forward(tokens)`` the (vocabulary-sharded) logits."""

    def __init__(self, cfg: MixtralConfig, dtype=torch.bfloat16):
        super().__init__()
        self.cfg = cfg
        self.tok_emb = Embedding(cfg.vocab, cfg.hidden, expert_mode=True, transpose=True,
                                 init_method=lambda w: nn.init.normal_(w, std=0.02), dtype=dtype)
        self.blocks = nn.ModuleList([MoEBlock(cfg, dtype) for _ in range(cfg.n_layers)])
        self.norm_f = TPNorm(cfg.hidden, cfg.eps, rms=True, dtype=dtype)
        self.head = ParallelLMHead(cfg.hidden, cfg.vocab, dtype=dtype)

    def forward(self, tokens, targets=None):
        x = self.tok_emb(tokens)
        delta = None   # expert-layer output of the previous block, added to x inside the next norm kernel
        for blk in self.blocks:
            if self.cfg.activation_checkpointing and self.training:
                if delta is not None:
                    x, delta = x + delta, None
                x = checkpoint(blk, x, use_reentrant=False)
            else:
                x, delta = blk.forward_deferred(x, delta)
        y = self.norm_f(x) if delta is None else self.norm_f.add_norm(x, delta)[1]
        out = self.head(y, targets)
        if targets is None:
            return out
        aux = sum(b.mlp.last_aux_loss for b in self.blocks) / len(self.blocks)
        return out + self.cfg.aux_loss_coef * aux.to(out.dtype)

    def num_parameters(self):
        return count_parameters(self)
