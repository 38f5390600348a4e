"""Intra-layer (tensor) parallelism: layers, collectives and gradient sync.

Public names match the reference's ``axonn/intra_layer/__init__.py`` plus the
two helpers its tests import but it never exported (``clear_weights_cache``,
``sync_gradients_depth_parallel``).
"""

from contextlib import contextmanager

import torch
import torch.distributed as dist

from .. import axonn as ax
from .. import ops
from .automatic_parallelism import auto_parallelize  # noqa: F401
from .communication import (  # noqa: F401
    BackwardAllReduce,
    Drop,
    ForwardAllReduce,
    ForwardGather_BackwardReduceScatter,
    Gather,
)
from .conv import Conv2d  # noqa: F401
from .embedding import Embedding  # noqa: F401
from .fully_connected import Linear  # noqa: F401
from .gradient_normalization import clip_grad_norm_  # noqa: F401
from .gradient_pruning import prune_gradients_, register_pruning_hooks  # noqa: F401
from .overlap_communication import (  # noqa: F401
    clear_weights_cache,
    optimize_communication,
    overlap_all_gathers_for_checkpointed_forward,
)

NO_GRADIENT_SYNC = False


@contextmanager
def no_grad_sync():
    """Suppress ``sync_gradients`` (gradient accumulation across microbatches)."""
    global NO_GRADIENT_SYNC
    old = NO_GRADIENT_SYNC
    NO_GRADIENT_SYNC = True
    try:
        yield None
    finally:
        NO_GRADIENT_SYNC = old


def _grads(model, attr):
    for p in model.parameters():
        if p.requires_grad:
            g = getattr(p, attr, None)
            if g is not None:
                yield p, g


def _needs_depth_sync(p):
    """True for parameters replicated over the depth group (TP biases, and every
    parameter that is not tensor parallel)."""
    if getattr(p, "is_tensor_parallel", False):
        return bool(getattr(p, "needs_depth_parallel_gradient_sync", False))
    return True


def _all_reduce_many(grads, group, scale=None, vectorize=False):
    """Sum ``grads`` over ``group`` (and multiply by ``scale``).

    On GPU the tensors travel as one flat bucket through the fused
    all-reduce+scale kernel; otherwise one collective per tensor (or one flat
    collective when ``vectorize``)."""
    if not grads:
        return
    n = dist.get_world_size(group)
    if n == 1:
        if scale is not None and scale != 1.0:
            ops.multi_tensor_scale_(grads, scale)
        return
    ops.all_reduce_bucketed_(grads, group, scale=scale, coalesce=vectorize or grads[0].is_cuda)


@torch.no_grad()
def sync_gradients_expert_mode_depth_parallel(model, gradient_attr_name="grad", mean=False, vectorize=False):
    """Depth-group reduction of gradients of depth-replicated parameters.  With
    ``mean`` every gradient is divided by the depth size (weights were already
    summed over depth by their reduce-scatter)."""
    if NO_GRADIENT_SYNC:
        return
    group = ax.comm_handle.depth_intra_layer_parallel_group
    n = dist.get_world_size(group)
    scale = 1.0 / n if mean else None
    synced, only_scaled = [], []
    for p, g in _grads(model, gradient_attr_name):
        (synced if _needs_depth_sync(p) else only_scaled).append(g)
    _all_reduce_many(synced, group, scale, vectorize)
    if scale is not None and only_scaled and n > 1:
        ops.multi_tensor_scale_(only_scaled, scale)


sync_gradients_depth_parallel = sync_gradients_expert_mode_depth_parallel


@torch.no_grad()
def sync_gradients_expert_mode_data_parallel(model, gradient_attr_name="grad", mean=False, vectorize=False):
    """Data-parallel reduction of every gradient except those of expert-parallel parameters (whose data-parallel
    ranks hold different experts); ``mean`` divides by the data-parallel size."""
    if NO_GRADIENT_SYNC:
        return
    group = ax.comm_handle.data_parallel_group
    n = dist.get_world_size(group)
    grads = [g for p, g in _grads(model, gradient_attr_name) if not getattr(p, "is_expert_parallel", False)]
    _all_reduce_many(grads, group, 1.0 / n if mean else None, vectorize)
    if mean and n > 1:
        # expert-parallel parameters live on one data-parallel rank only: no
        # sum, but the same 1/n so that all parameters see the global mean
        ep = [g for p, g in _grads(model, gradient_attr_name) if getattr(p, "is_expert_parallel", False)]
        if ep:
            ops.multi_tensor_scale_(ep, 1.0 / n)


@torch.no_grad()
def sync_gradients(model, gradient_attr_name="grad", mean=False, vectorize=False, expert_mode=False):
    """Sum (or average) gradients over the replicas of each parameter.

    expert_mode=True: depth group for depth-replicated parameters, then data
    group for all; ``mean`` divides by the two group sizes.
    expert_mode=False ("easy"): TP weights over data; TP biases over data and
    depth; every other parameter over the whole world; ``mean`` divides by the
    world size (each rank saw a different batch shard).  Expert-parallel
    parameters (``is_expert_parallel``) are summed over the tensor-parallel grid
    only and get the same 1/world scale.
    Reference: ``axonn/intra_layer/__init__.py:114-173``."""
    if NO_GRADIENT_SYNC:
        return
    if expert_mode:
        sync_gradients_expert_mode_depth_parallel(model, gradient_attr_name, mean, vectorize)
        sync_gradients_expert_mode_data_parallel(model, gradient_attr_name, mean, vectorize)
        return
    ch = ax.comm_handle
    weights, biases, others, experts = [], [], [], []
    for p, g in _grads(model, gradient_attr_name):
        if getattr(p, "is_expert_parallel", False):
            # a different expert on every data-parallel rank: summed over the replicas inside the
            # tensor-parallel grid only, never over the data group (that would mix unrelated experts)
            experts.append(g)
        elif getattr(p, "is_tensor_parallel", False):
            if not hasattr(p, "needs_depth_parallel_gradient_sync"):
                raise ValueError("tensor-parallel parameter without needs_depth_parallel_gradient_sync")
            (biases if p.needs_depth_parallel_gradient_sync else weights).append(g)
        else:
            others.append(g)
    scale = 1.0 / dist.get_world_size() if mean else None
    _all_reduce_many(weights, ch.data_parallel_group, scale, vectorize)
    _all_reduce_many(biases, ch.data_parallel_group, None, vectorize)
    _all_reduce_many(biases, ch.depth_intra_layer_parallel_group, scale, vectorize)
    _all_reduce_many(others, dist.group.WORLD, scale, vectorize)
    _all_reduce_many(experts, ch.intra_layer_group, scale, vectorize)
