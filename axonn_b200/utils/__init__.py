"""Small helpers shared across the package."""

from typing import List

import torch
from torch._utils import _flatten_dense_tensors, _unflatten_dense_tensors


def divide(a: int, b: int) -> int:
    if a % b != 0:
        raise ValueError(f"{a} is not divisible by {b}")
    return a // b


def coalesce_and_reassign(tensors: List[torch.Tensor]) -> torch.Tensor:
    """Flatten ``tensors`` into one buffer and re-point each at its slice
    (same service as the reference's ``axonn/utils.py:_coalesce_and_reassign``)."""
    flat = _flatten_dense_tensors(tensors)
    for old, new in zip(tensors, _unflatten_dense_tensors(flat, tensors)):
        old.data = new
    return flat


def print_rank0(*args, **kwargs):
    import torch.distributed as dist

    if not dist.is_initialized() or dist.get_rank() == 0:
        print(*args, **kwargs, flush=True)
