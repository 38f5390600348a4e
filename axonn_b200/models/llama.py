"""Llama-style decoder: RMSNorm, rotary embeddings, grouped-query attention,
SwiGLU MLP, no biases.  ``LlamaConfig.llama_8b()`` is the 8B configuration
(32 layers, d_model 4096, 32 query / 8 KV heads, FFN 14336, vocabulary 128256,
sequence 4096, rope theta 500000).

Replaces the HF monkey patch ``axonn/models/transformers/modify_llama.py`` of
the reference with a native definition on this package's layers and kernels.
"""

from dataclasses import dataclass

import torch
import torch.nn as nn
from torch.utils.checkpoint import checkpoint

from ..intra_layer import Embedding
from .blocks import ParallelLMHead, TPNorm, TransformerBlock, count_parameters


@dataclass
class LlamaConfig:
    """Shape of a Llama-style model; ``llama_8b()`` is the benchmark configuration, ``tiny()`` the test one."""

    n_layers: int = 32
    hidden: int = 4096
    n_heads: int = 32
    n_kv_heads: int = 8
    ffn: int = 14336
    vocab: int = 128256
    seq_len: int = 4096
    rope_theta: float = 500000.0
    eps: float = 1e-5
    activation_checkpointing: bool = False

    @staticmethod
    def llama_8b(**kw):
        return LlamaConfig(**kw)

    @staticmethod
    def tiny(**kw):
        return LlamaConfig(n_layers=2, hidden=128, n_heads=4, n_kv_heads=2, ffn=256, vocab=512, seq_len=64, **kw)

    def flops_per_token(self):
        h, L = self.hidden, self.n_layers
        hd = h // self.n_heads
        per_layer = 2 * h * h + 2 * h * self.n_kv_heads * hd + 3 * h * self.ffn
        return 6 * (L * per_layer + h * self.vocab) + 6 * L * self.seq_len * h


class Llama(nn.Module):
    """Decoder-only transformer with RMSNorm, rotary grouped-query attention and SwiGLU feed-forward layers on the
    tensor-parallel building blocks; ``forward(tokens, targets)`` returns the loss, ``forward(tokens)`` the
    (vocabulary-sharded) logits."""

    def __init__(self, cfg: LlamaConfig, dtype=torch.bfloat16):
        super().__init__()
        self.cfg = cfg
        self.tok_emb = Embedding(cfg.vocab, cfg.hidden, expert_mode=True, transpose=True,
                                 init_method=lambda w: nn.init.normal_(w, std=0.02), dtype=dtype)
        self.blocks = nn.ModuleList([
            TransformerBlock(cfg.hidden, cfg.n_heads, cfg.ffn, n_kv_heads=cfg.n_kv_heads, activation="swiglu",
                             rms=True, bias=False, rope_theta=cfg.rope_theta, max_seq=cfg.seq_len, eps=cfg.eps,
                             dtype=dtype, n_layers=cfg.n_layers)
            for _ in range(cfg.n_layers)])
        self.norm_f = TPNorm(cfg.hidden, cfg.eps, rms=True, dtype=dtype)
        self.head = ParallelLMHead(cfg.hidden, cfg.vocab, dtype=dtype)

    def forward(self, tokens, targets=None):
        x = self.tok_emb(tokens)
        delta = None   # MLP output of the previous block, added to x inside the next norm kernel
        for blk in self.blocks:
            if self.cfg.activation_checkpointing and self.training:
                if delta is not None:
                    x, delta = x + delta, None
                x = checkpoint(blk, x, use_reentrant=False)
            else:
                x, delta = blk.forward_deferred(x, delta)
        y = self.norm_f(x) if delta is None else self.norm_f.add_norm(x, delta)[1]
        return self.head(y, targets)

    def num_parameters(self):
        return count_parameters(self)
