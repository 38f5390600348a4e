"""GPT-style decoder (LayerNorm, learned positions, GELU MLP) on the
tensor-parallel layers.  The 1.3B configuration is ``GPTConfig.gpt_1p3b()``:
24 layers, d_model 2048, 16 heads, FFN 8192, vocabulary 50304, sequence 2048.

Own model definition standing in for ``external/models/nvidia_transformer.py``
(Megatron-based, not importable upstream) of the reference.
"""

from dataclasses import dataclass

import torch
import torch.nn as nn
from torch.utils.checkpoint import checkpoint

from .. import axonn as ax
from ..intra_layer import Embedding
from .blocks import ParallelLMHead, TPNorm, TransformerBlock, count_parameters


@dataclass
class GPTConfig:
    n_layers: int = 24
    hidden: int = 2048
    n_heads: int = 16
    ffn: int = 8192
    vocab: int = 50304
    seq_len: int = 2048
    activation_checkpointing: bool = False

    @staticmethod
    def gpt_1p3b(**kw):
        return GPTConfig(**kw)

    @staticmethod
    def tiny(**kw):
        return GPTConfig(n_layers=2, hidden=128, n_heads=4, ffn=512, vocab=512, seq_len=64, **kw)

    def flops_per_token(self):
        """Model FLOPs per token for forward+backward (6 N + attention term)."""
        h, L = self.hidden, self.n_layers
        per_layer = 4 * h * h + 2 * h * self.ffn
        dense = 6 * (L * per_layer + h * self.vocab)
        attn = 6 * L * self.seq_len * h  # causal: half of 12 * L * S * h
        return dense + attn


class GPT(nn.Module):
    def __init__(self, cfg: GPTConfig, dtype=torch.bfloat16):
        super().__init__()
        self.cfg = cfg
        init = lambda w: nn.init.normal_(w, std=0.02)  # noqa: E731
        self.tok_emb = Embedding(cfg.vocab, cfg.hidden, expert_mode=True, transpose=True, init_method=init,
                                 dtype=dtype)
        self.pos_emb = Embedding(cfg.seq_len, cfg.hidden, expert_mode=True, transpose=True, init_method=init,
                                 dtype=dtype)
        self.blocks = nn.ModuleList([
            TransformerBlock(cfg.hidden, cfg.n_heads, cfg.ffn, activation="gelu", rms=False, bias=True,
                             max_seq=cfg.seq_len, dtype=dtype, n_layers=cfg.n_layers)
            for _ in range(cfg.n_layers)])
        self.norm_f = TPNorm(cfg.hidden, dtype=dtype)
        self.head = ParallelLMHead(cfg.hidden, cfg.vocab, dtype=dtype)

    def forward(self, tokens, targets=None):
        B, S = tokens.shape
        pos = torch.arange(S, device=tokens.device)
        x = self.tok_emb(tokens) + self.pos_emb(pos)[None]
        for blk in self.blocks:
            if self.cfg.activation_checkpointing and self.training:
                x = checkpoint(blk, x, use_reentrant=False)
            else:
                x = blk(x)
        return self.head(self.norm_f(x), targets)

    def num_parameters(self):
        return count_parameters(self)
