"""Two-layer MLP from tensor-parallel ``Linear`` layers (the smallest end-to-end
model; runs on CPU ranks with gloo)."""

import torch.nn as nn

from ..intra_layer import Linear


class MLP(nn.Module):
    """Two tensor-parallel ``Linear`` layers with a GELU between them (the smallest model that exercises every
    collective of the 3-D algorithm)."""

    def __init__(self, d_in=1024, d_hidden=4096, d_out=1024, expert_mode=True, dtype=None):
        super().__init__()
        self.fc1 = Linear(d_in, d_hidden, expert_mode=expert_mode, dtype=dtype)
        self.act = nn.GELU()
        self.fc2 = Linear(d_hidden, d_out, expert_mode=expert_mode, transpose=True, dtype=dtype)

    def forward(self, x):
        return self.fc2(self.act(self.fc1(x)))
