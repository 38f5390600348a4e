"""``auto_parallelize``: build tensor-parallel layers from unmodified model code.

Inside the context ``torch.nn.Linear(...)`` returns this package's ``Linear``
whenever the shape divides the grid (``out % G_r == 0``, ``in % G_c == 0`` and
the local block divides by ``G_d``), and the stock class otherwise — the
contract of the reference's ``axonn/intra_layer/automatic_parallelism.py``.
``torch.nn.Embedding`` is patched the same way when ``embeddings=True``
(the reference has that patch commented out, ``:90-96``).
"""

from contextlib import contextmanager

import torch.nn as nn

from .. import axonn as ax
from .embedding import Embedding
from .fully_connected import Linear

_original_linear = nn.Linear
_original_embedding = nn.Embedding


def is_parallelizable_linear(in_features, out_features):
    """``out`` divisible by the row size, ``in`` by the column size, and the local block by the depth size."""
    c = ax.config
    return (out_features % c.G_intra_r == 0 and in_features % c.G_intra_c == 0
            and (out_features * in_features // (c.G_intra_r * c.G_intra_c)) % c.G_intra_d == 0)


def is_parallelizable_embedding(num_embeddings, embedding_dim):
    c = ax.config
    return (embedding_dim % c.G_intra_r == 0 and c.G_intra_c == 1
            and (num_embeddings * embedding_dim // c.G_intra_r) % c.G_intra_d == 0)


def _place(layer, device, dtype):
    if device is not None:
        layer = layer.to(device)
    if dtype is not None:
        layer = layer.to(dtype)
    return layer


class patched_linear:
    def __new__(cls, in_features, out_features, *args, bias=True, device=None, dtype=None, **kwargs):
        if is_parallelizable_linear(in_features, out_features):
            layer = Linear(in_features, out_features, *args, bias=bias, **kwargs)
        else:
            layer = _original_linear(in_features, out_features, *args, bias=bias, **kwargs)
        return _place(layer, device, dtype)


class patched_embedding:
    def __new__(cls, num_embeddings, embedding_dim, *args, device=None, dtype=None, **kwargs):
        if is_parallelizable_embedding(num_embeddings, embedding_dim):
            layer = Embedding(num_embeddings, embedding_dim, *args, **kwargs)
        else:
            layer = _original_embedding(num_embeddings, embedding_dim, *args, **kwargs)
        return _place(layer, device, dtype)


@contextmanager
def auto_parallelize(embeddings=False):
    """Context manager under which ``torch.nn.Linear(...)`` builds a tensor-parallel ``Linear`` (easy mode)
    whenever the shape divides the grid (:func:`is_parallelizable_linear`), and the plain layer otherwise;
    ``embeddings=True`` does the same for ``torch.nn.Embedding``.  ``device`` and ``dtype`` arguments are applied
    to the new layer (reference ``axonn/intra_layer/automatic_parallelism.py:15-96``)."""
    nn.Linear = patched_linear
    if embeddings:
        nn.Embedding = patched_embedding
    try:
        yield None
    finally:
        nn.Linear = _original_linear
        nn.Embedding = _original_embedding
