"""Token-stream datasets for language-model training.

The upstream examples read WikiText and Penn Treebank through their own loaders
(``examples/wikitext_loader.py:14-62``, ``examples/ptb_loader.py:11-57``: tokenise, concatenate, cut into
fixed-length windows).  ``TokenWindows`` is that last step for any source of token ids, and ``load_tokens`` turns
the common on-disk forms into such a source without a tokenizer dependency:

* ``.npy`` / ``.bin`` (raw little-endian ``uint16`` or ``int32``) files of token ids, memory-mapped;
* any other file, read as bytes (a byte-level vocabulary of 256 symbols).
"""

import os
from typing import Optional

import numpy as np
import torch


def load_tokens(path: str, dtype: Optional[str] = None) -> np.ndarray:
    """Token ids of ``path`` as a 1-D array (memory-mapped where the format allows it)."""
    ext = os.path.splitext(path)[1].lower()
    if ext == ".npy":
        return np.load(path, mmap_mode="r").reshape(-1)
    if ext == ".bin":
        return np.memmap(path, dtype=np.dtype(dtype or "uint16"), mode="r")
    return np.memmap(path, dtype=np.uint8, mode="r")


class TokenWindows(torch.utils.data.Dataset):
    """Windows of ``seq_len + 1`` consecutive tokens, returned as ``(inputs, targets)`` shifted by one position.

    Windows start every ``stride`` tokens (default ``seq_len``: no overlap).  ``vocab`` (optional) is checked
    against the largest id of the stream once, at construction."""

    def __init__(self, tokens, seq_len: int, stride: Optional[int] = None, vocab: Optional[int] = None):
        self.tokens = tokens
        self.seq_len = int(seq_len)
        self.stride = int(stride or seq_len)
        n = len(tokens)
        if n < self.seq_len + 1:
            raise ValueError(f"{n} tokens are fewer than one window of {self.seq_len + 1}")
        self.count = (n - self.seq_len - 1) // self.stride + 1
        if vocab is not None:
            top = int(np.max(tokens)) if not torch.is_tensor(tokens) else int(tokens.max())
            if top >= vocab:
                raise ValueError(f"token id {top} does not fit a vocabulary of {vocab}")

    def __len__(self):
        return self.count

    def __getitem__(self, i):
        if not 0 <= i < self.count:
            raise IndexError(i)
        a = i * self.stride
        w = self.tokens[a:a + self.seq_len + 1]
        w = w.to(torch.long) if torch.is_tensor(w) else torch.from_numpy(np.asarray(w).astype(np.int64))
        return w[:-1], w[1:]
