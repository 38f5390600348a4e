"""GPT-style decoder (LayerNorm, learned positions, GELU MLP) on the
tensor-parallel layers.  The 1.3B configuration is ``GPTConfig.gpt_1p3b()``:
24 layers, d_model 2048, 16 heads, FFN 8192, vocabulary 50304, sequence 2048.

Own model definition standing in for ``external/models/nvidia_transformer.py``
(Megatron-based, not importable upstream) of the reference.
"""

from dataclasses import dataclass

import torch
import torch.distributed as dist
import torch.nn as nn
from torch.utils.checkpoint import checkpoint

from .. import axonn as ax
from ..intra_layer import Embedding
from .blocks import ParallelLMHead, TPNorm, TransformerBlock, count_parameters


@dataclass
class GPTConfig:
    """Shape of a GPT-style model; ``gpt_1p3b()`` is the benchmark configuration, ``tiny()`` the test one."""

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
    """Decoder-only transformer with learned positions, LayerNorm and GELU feed-forward layers on the
    tensor-parallel building blocks; ``forward(tokens, targets)`` returns the loss, ``forward(tokens)`` the
    (vocabulary-sharded) logits."""

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
        self.sequence_group = None     # set by parallel.sequence.enable_sequence_parallel

    def forward(self, tokens, targets=None):
        B, S = tokens.shape
        pos = torch.arange(S, device=tokens.device)
        if self.sequence_group is not None:
            pos = pos + dist.get_rank(self.sequence_group) * S      # this rank's slice of the positions
        x = self.tok_emb(tokens) + self.pos_emb(pos)[None]
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


class DistributedGPT(nn.Module):
    """One pipeline stage of the GPT above, for the inter-layer engine.

    Stage ``s`` of ``G_inter`` owns ``n_layers // G_inter`` consecutive blocks; the first stage also owns the
    token / position embeddings, the last one the final norm and the LM head (logits out; the engine's loss
    function gets ``[microbatch, seq, vocab_local]``).  Activation checkpointing wraps every ``ckp_coeff``
    blocks when enabled.  ``get_input_shape`` / ``get_output_shape`` use ``-1`` for the microbatch dimension,
    which is the engine's contract.  Same role as ``DistributedGPT`` in
    ``external/models/nvidia_transformer.py`` of the reference (there ``[seq, -1, hidden]``; here
    batch-first ``[-1, seq, hidden]``, the layout of this package's attention kernels).
    """

    def __init__(self, cfg: GPTConfig, dtype=torch.bfloat16, ckp_coeff=1, G_inter=None, stage=None):
        super().__init__()
        G_inter = ax.config.G_inter if G_inter is None else G_inter
        stage = ax.config.inter_layer_parallel_rank if stage is None else stage
        assert cfg.n_layers % G_inter == 0, "n_layers must be divisible by the number of pipeline stages"
        self.cfg, self.ckp_coeff = cfg, max(1, int(ckp_coeff))
        self.first, self.last = stage == 0, stage == G_inter - 1
        init = lambda w: nn.init.normal_(w, std=0.02)  # noqa: E731
        if self.first:
            self.tok_emb = Embedding(cfg.vocab, cfg.hidden, expert_mode=True, transpose=True, init_method=init,
                                     dtype=dtype)
            self.pos_emb = Embedding(cfg.seq_len, cfg.hidden, expert_mode=True, transpose=True, init_method=init,
                                     dtype=dtype)
        self.blocks = nn.ModuleList([
            TransformerBlock(cfg.hidden, cfg.n_heads, cfg.ffn, activation="gelu", rms=False, bias=True,
                             max_seq=cfg.seq_len, dtype=dtype, n_layers=cfg.n_layers)
            for _ in range(cfg.n_layers // G_inter)])
        if self.last:
            self.norm_f = TPNorm(cfg.hidden, dtype=dtype)
            self.head = ParallelLMHead(cfg.hidden, cfg.vocab, dtype=dtype)
        self._dtype = dtype

    def _hidden_local(self):
        return self.blocks[0].norm1.local

    def get_input_shape(self):
        if self.first:
            return [-1, self.cfg.seq_len]
        return [-1, self.cfg.seq_len, self._hidden_local()]

    def get_output_shape(self):
        if self.last:
            return [-1, self.cfg.seq_len, self.head.proj.local_out_features]
        return [-1, self.cfg.seq_len, self._hidden_local()]

    def input_dtype(self):
        return torch.long if self.first else self._dtype

    def _run_blocks(self, x, lo, hi):
        for blk in self.blocks[lo:hi]:
            x = blk(x)
        return x

    def forward(self, x):
        if self.first:
            tokens = x.long()
            pos = torch.arange(tokens.shape[1], device=tokens.device)
            x = self.tok_emb(tokens) + self.pos_emb(pos)[None]
        n = len(self.blocks)
        for lo in range(0, n, self.ckp_coeff):
            hi = min(n, lo + self.ckp_coeff)
            if self.cfg.activation_checkpointing and self.training:
                x = checkpoint(self._run_blocks, x, lo, hi, use_reentrant=False)
            else:
                x = self._run_blocks(x, lo, hi)
        if self.last:
            x = self.head(self.norm_f(x))
        return x
