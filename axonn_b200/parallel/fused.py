"""Python entry points of the fused compute+collective kernels.

Each ``try_*`` function returns ``False`` when the fused path does not apply
(CPU tensors, ``AXONN_BACKEND=nccl``, group of one); the caller then runs the
collective through ``torch.distributed``.
"""

import torch
import torch.distributed as dist

from . import symm


def try_all_reduce_scale_(grads, group, scale) -> bool:
    return False
