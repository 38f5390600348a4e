"""Global gradient-norm clipping over sharded parameters.

Semantics of the reference's ``axonn/intra_layer/gradient_normalization.py``:
local p-norms are grouped by each parameter's
``process_group_for_norm_reduction``, ``norm**p`` is all-reduced per group,
combined with the norm of non-tensor-parallel parameters, and all gradients are
scaled by ``min(1, max_norm / (total + 1e-6))``.  The per-tensor norms come
from one multi-tensor kernel on GPU (``ops.multi_tensor_l2norm_sq``) and the
infinity norm is supported as well (not implemented upstream, ``:40-41``).
"""

from collections import defaultdict
from math import inf

import torch
import torch.distributed as dist

from .. import ops


def _local_norm_pow(grads, norm_type):
    """sum_i ||g_i||_p^p as an fp32 scalar tensor (max for p=inf)."""
    if not grads:
        return None
    if norm_type == inf:
        return torch.stack([g.detach().abs().max().float() for g in grads]).max()
    if norm_type == 2.0:
        return ops.multi_tensor_l2norm_sq(grads)
    return torch.stack([torch.linalg.vector_norm(g.detach().float(), norm_type) ** norm_type
                        for g in grads]).sum()


def clip_grad_norm_(parameters, max_norm, norm_type=2.0, error_if_nonfinite=False):
    """``torch.nn.utils.clip_grad_norm_`` for sharded parameters: the local norms of tensor-parallel parameters
    are reduced over ``param.process_group_for_norm_reduction`` (replicas counted once), combined with the norm
    of the replicated parameters, and every gradient is scaled by ``min(1, max_norm / (total + 1e-6))``.  Any
    ``norm_type`` > 0 including ``inf``; returns the total norm (reference
    ``axonn/intra_layer/gradient_normalization.py:18-95``, which has no ``inf`` norm)."""
    if isinstance(parameters, torch.Tensor):
        parameters = [parameters]
    parameters = list(parameters)
    max_norm, norm_type = float(max_norm), float(norm_type)
    by_group, plain = defaultdict(list), []
    for p in parameters:
        if p.grad is None:
            continue
        if getattr(p, "is_tensor_parallel", False):
            assert hasattr(p, "process_group_for_norm_reduction"), (
                "tensor-parallel parameters need process_group_for_norm_reduction")
            # a shard that is held by several ranks of its reduction group (e.g. an
            # embedding replicated over the row group) must count once
            replicas = int(getattr(p, "norm_reduction_replicas", 1))
            by_group[(p.process_group_for_norm_reduction, replicas)].append(p.grad)
        else:
            plain.append(p.grad)
    pieces = []
    for (group, replicas), grads in by_group.items():
        v = _local_norm_pow(grads, norm_type)
        if replicas > 1 and norm_type != inf:
            v = v / replicas
        if dist.get_world_size(group) > 1:
            dist.all_reduce(v, op=dist.ReduceOp.MAX if norm_type == inf else dist.ReduceOp.SUM, group=group)
        pieces.append(v)
    v = _local_norm_pow(plain, norm_type)
    if v is not None:
        pieces.append(v)
    if not pieces:
        return torch.tensor(0.0)
    dev = pieces[0].device
    pieces = torch.stack([p.to(dev) for p in pieces])
    total_norm = pieces.max() if norm_type == inf else pieces.sum() ** (1.0 / norm_type)
    if error_if_nonfinite and total_norm.is_cuda:
        finite = bool(torch.isfinite(total_norm))   # host synchronisation: every kernel before it has finished
        from ..ops import _lib

        _lib.check_status(total_norm.device.index)   # an expired device-side wait surfaces here, not silently
    else:
        finite = (not error_if_nonfinite) or bool(torch.isfinite(total_norm))
    if not finite:
        raise RuntimeError(f"The total norm of order {norm_type} for gradients is non-finite, "
                           "so it cannot be clipped.")
    clip = torch.clamp(max_norm / (total_norm + 1e-6), max=1.0)
    all_grads = plain + [g for gs in by_group.values() for g in gs]
    ops.multi_tensor_scale_(all_grads, clip)
    return total_norm
