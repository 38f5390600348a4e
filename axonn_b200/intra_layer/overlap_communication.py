"""Communication-overlap policy and its per-step state.

API of the reference's ``axonn/intra_layer/overlap_communication.py:11-159``:
``optimize_communication(...)`` selects which collectives of the
tensor-parallel layers run asynchronously, and
``overlap_all_gathers_for_checkpointed_forward`` re-targets the depth
all-gather prefetcher for recompute/backward order.

What differs here:

* ``cache_weights`` is a real parameter: with it the depth-gathered weight of
  each layer is kept from forward to backward, so backward issues no second
  all-gather (the reference swallows the keyword, ``:125-132``);
* outstanding work is tracked as handles and waited individually at context
  exit; there is no device-wide synchronize (reference ``:27-30``);
* gradient pieces produced by asynchronous reduce-scatters are added to
  ``param.grad`` at exit, exactly like the reference (``:33-47``), so the
  observable contract "``.grad`` is complete after the ``with`` block" holds.
"""

from contextlib import contextmanager

import torch
import torch.distributed as dist

OVERLAP_REDUCE_SCATTER = False
OVERLAP_ALL_REDUCE = False
CACHE_WEIGHTS = False
ALL_GATHER_ITERATOR = None

handles = []
pending_grad_accumulations = []
# id(param) -> [param, gathered weight, handle or None]; keyed by id so the
# lookup does not hash tensor contents and keeps the parameter alive.
weights_cache = {}


def reset_state():
    global OVERLAP_ALL_REDUCE, OVERLAP_REDUCE_SCATTER, CACHE_WEIGHTS, ALL_GATHER_ITERATOR
    global handles, pending_grad_accumulations, weights_cache
    OVERLAP_ALL_REDUCE = OVERLAP_REDUCE_SCATTER = CACHE_WEIGHTS = False
    ALL_GATHER_ITERATOR = None
    handles, pending_grad_accumulations, weights_cache = [], [], {}


def register_handle(handle):
    if handle is not None:
        handles.append(handle)


def clear_handles():
    """Wait for every registered asynchronous collective (stream-level wait on
    GPU: the host does not block)."""
    global handles
    for h in handles:
        h.wait()
    handles = []


def accumulate_later(param, grad):
    pending_grad_accumulations.append((param, grad))


@torch.no_grad()
def accumulate():
    global pending_grad_accumulations
    for param, grad in pending_grad_accumulations:
        g = grad.to(param.dtype).reshape(param.shape)
        if param.grad is None:
            param.grad = g.contiguous()
        else:
            param.grad.add_(g)
    pending_grad_accumulations = []


def clear_weights_cache():
    """Drop the all-gathered weights kept by ``cache_weights`` / the prefetcher."""
    global weights_cache
    weights_cache = {}


def _tp_layer_types():
    from .fully_connected import Linear
    from .conv import Conv2d
    from .embedding import Embedding

    return (Linear, Conv2d, Embedding)


def launch_all_gather(weight, process_group):
    """Start an asynchronous depth all-gather of a flat weight shard and put it
    in the cache; returns the cache entry."""
    world = dist.get_world_size(process_group)
    if world == 1:
        entry = [weight, weight, None]
    else:
        assert weight.ndim == 1
        full = torch.empty(weight.shape[0] * world, dtype=weight.dtype, device=weight.device)
        h = dist.all_gather_into_tensor(full, weight.detach().contiguous(), group=process_group, async_op=True)
        entry = [weight, full, h]
    weights_cache[id(weight)] = entry
    return entry


def trigger_async_all_gathers(model_or_modules):
    """Generator: each ``next`` starts the depth all-gather of one more
    tensor-parallel layer, in the order the modules are given."""
    types = _tp_layer_types()
    if isinstance(model_or_modules, torch.nn.Module):
        modules = model_or_modules.modules()
    else:
        modules = model_or_modules
    for module in modules:
        if isinstance(module, types):
            weight = module.weight
            if id(weight) not in weights_cache:
                launch_all_gather(weight, module.depth_group)
                yield


def enqueue_next_all_gather():
    if ALL_GATHER_ITERATOR is None:
        return
    try:
        next(ALL_GATHER_ITERATOR)
    except StopIteration:
        pass


def retrieve_all_gathered_weight(weight, delete):
    """Pop (or peek) a gathered weight; consuming one schedules the next
    prefetch (one layer of look-ahead, reference ``:91-99``)."""
    entry = weights_cache[id(weight)]
    enqueue_next_all_gather()
    if delete:
        del weights_cache[id(weight)]
    return entry[1], entry[2]


@contextmanager
def overlap_all_gathers_for_checkpointed_forward(model_object_for_overlapping_allgathers):
    """Inside ``optimize_communication(overlap_all_gather=True)``: prefetch in
    the order of the given modules (e.g. a checkpointed block about to be
    recomputed, or the layers in reverse for backward)."""
    global ALL_GATHER_ITERATOR
    if ALL_GATHER_ITERATOR is None:
        yield None
        return
    old = ALL_GATHER_ITERATOR
    ALL_GATHER_ITERATOR = trigger_async_all_gathers(model_object_for_overlapping_allgathers)
    enqueue_next_all_gather()
    try:
        yield None
    finally:
        ALL_GATHER_ITERATOR = old


@contextmanager
def optimize_communication(
    overlap_all_reduce=True,
    overlap_reduce_scatter=False,
    cache_weights=False,
    overlap_all_gather=False,
    model_object_for_overlapping_allgathers=None,
    *args,
    **kwargs,
):
    """Select overlap optimisations for the enclosed forward/backward.

    overlap_all_reduce      backward activation-gradient all-reduce (outer
                            group) runs under the weight-gradient GEMM
    overlap_reduce_scatter  depth reduce-scatter of weight gradients runs
                            asynchronously; results land in ``.grad`` at exit
    cache_weights           keep each layer's depth-gathered weight from its
                            forward until its backward
    overlap_all_gather      prefetch the next layer's depth all-gather while
                            the current layer computes (needs the model)
    """
    global OVERLAP_ALL_REDUCE, OVERLAP_REDUCE_SCATTER, CACHE_WEIGHTS, ALL_GATHER_ITERATOR
    OVERLAP_ALL_REDUCE = overlap_all_reduce
    OVERLAP_REDUCE_SCATTER = overlap_reduce_scatter
    CACHE_WEIGHTS = cache_weights
    if overlap_all_gather:
        if model_object_for_overlapping_allgathers is None:
            raise ValueError(
                "overlap_all_gather=True needs the model: optimize_communication(..., "
                "model_object_for_overlapping_allgathers=model)"
            )
        ALL_GATHER_ITERATOR = trigger_async_all_gathers(model_object_for_overlapping_allgathers)
        enqueue_next_all_gather()
    try:
        yield None
    finally:
        clear_handles()
        accumulate()
        clear_weights_cache()
        OVERLAP_ALL_REDUCE = False
        OVERLAP_REDUCE_SCATTER = False
        CACHE_WEIGHTS = False
        ALL_GATHER_ITERATOR = None
