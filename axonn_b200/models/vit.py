"""Vision Transformer split into pipeline stages.

``DistributedViT`` holds ``depth // G_inter`` encoder layers per stage; the
first stage owns patch embedding, class token and positions, the last stage
owns the classification head.  It implements the stage contract of the
pipeline engine (``get_input_shape`` / ``get_output_shape`` with ``-1`` for the
microbatch dimension).  Same role as the reference's
``external/models/vit.py:121-217``.
"""

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import axonn as ax


class _EncoderLayer(nn.Module):
    def __init__(self, dim, heads, mlp_dim, dropout=0.0):
        super().__init__()
        self.heads = heads
        self.norm1, self.norm2 = nn.LayerNorm(dim), nn.LayerNorm(dim)
        self.qkv, self.proj = nn.Linear(dim, 3 * dim), nn.Linear(dim, dim)
        self.fc1, self.fc2 = nn.Linear(dim, mlp_dim), nn.Linear(mlp_dim, dim)
        self.drop = nn.Dropout(dropout)

    def forward(self, x):
        B, N, C = x.shape
        qkv = self.qkv(self.norm1(x)).view(B, N, 3, self.heads, C // self.heads).permute(2, 0, 3, 1, 4)
        a = F.scaled_dot_product_attention(qkv[0], qkv[1], qkv[2])
        x = x + self.drop(self.proj(a.transpose(1, 2).reshape(B, N, C)))
        return x + self.drop(self.fc2(F.gelu(self.fc1(self.norm2(x)))))


class DistributedViT(nn.Module):
    """One pipeline stage of a vision transformer: ``depth // G_inter`` encoder layers; the first stage also owns
    patch embedding, class token and positions, the last one the classification head.  ``get_input_shape()`` /
    ``get_output_shape()`` give the engine the shapes of the tensors that travel between stages (``-1`` = the
    microbatch dimension) - the contract of the upstream ``external/models/vit.py:121-217``."""

    def __init__(self, *, image_size, patch_size, num_classes, dim, depth, heads, mlp_dim, channels=3,
                 dropout=0.0, G_inter=None, stage=None):
        super().__init__()
        G_inter = ax.config.G_inter if G_inter is None else G_inter
        stage = ax.config.inter_layer_parallel_rank if stage is None else stage
        assert depth % G_inter == 0, "depth must be divisible by the number of pipeline stages"
        assert image_size % patch_size == 0
        self.first, self.last = stage == 0, stage == G_inter - 1
        self.num_patches = (image_size // patch_size) ** 2
        self.dim, self.channels, self.image_size, self.num_classes = dim, channels, image_size, num_classes
        self.patch_size = patch_size
        if self.first:
            self.patch_embed = nn.Linear(channels * patch_size * patch_size, dim)
            self.cls_token = nn.Parameter(torch.randn(1, 1, dim) * 0.02)
            self.pos_embedding = nn.Parameter(torch.randn(1, self.num_patches + 1, dim) * 0.02)
        self.layers = nn.ModuleList([_EncoderLayer(dim, heads, mlp_dim, dropout) for _ in range(depth // G_inter)])
        if self.last:
            self.head = nn.Sequential(nn.LayerNorm(dim), nn.Linear(dim, num_classes))

    def get_input_shape(self):
        if self.first:
            return [-1, self.channels, self.image_size, self.image_size]
        return [-1, self.num_patches + 1, self.dim]

    def get_output_shape(self):
        if self.last:
            return [-1, self.num_classes]
        return [-1, self.num_patches + 1, self.dim]

    def forward(self, x):
        if self.first:
            B, C, H, W = x.shape
            p = self.patch_size
            x = x.view(B, C, H // p, p, W // p, p).permute(0, 2, 4, 3, 5, 1).reshape(B, -1, p * p * C)
            x = self.patch_embed(x)
            x = torch.cat([self.cls_token.expand(B, -1, -1).to(x.dtype), x], 1) + self.pos_embedding.to(x.dtype)
        for layer in self.layers:
            x = layer(x)
        if self.last:
            x = self.head(x[:, 0])
        return x
