"""Magnitude (top-k) gradient pruning of tensor-parallel weight shards.

Before the data-parallel reduction only the ``keep_fraction`` largest-magnitude entries of every selected
gradient shard are kept; the rest are set to zero in place.  The selection runs on the shard each rank owns
(``Linear`` weights are flat depth shards), so no communication is involved.  On CUDA the work is done by the
package's radix-select kernel (``ops.prune_topk_``: histogram passes over the key bits, then one masking
pass); on CPU by ``torch.kthvalue``.

The reference has no such component; it exists for the Llama depth-parallel + pruning configuration and is
wired either explicitly (``prune_gradients_`` between backward and ``sync_gradients``) or through
post-accumulate hooks (``register_pruning_hooks``), which prune each gradient as soon as autograd has
finished accumulating it so that the work overlaps the rest of the backward pass.
"""

from typing import Callable, Iterable, List, Optional

import torch

from .. import ops


def _default_filter(name: str, p: torch.nn.Parameter) -> bool:
    # matrices only: biases, norm gains and embeddings keep dense gradients
    return p.dim() >= 1 and getattr(p, "is_tensor_parallel", False) and not getattr(
        p, "needs_depth_parallel_gradient_sync", False) and "emb" not in name


def _selected(model: torch.nn.Module, param_filter: Optional[Callable]) -> List[torch.nn.Parameter]:
    flt = param_filter or _default_filter
    return [p for n, p in model.named_parameters() if p.requires_grad and flt(n, p)]


def prune_gradients_(model: torch.nn.Module, keep_fraction: float, gradient_attr_name: str = "grad",
                     param_filter: Optional[Callable] = None) -> int:
    """Prune the gradients of the selected parameters of ``model`` in place; returns how many were pruned."""
    assert 0.0 < keep_fraction <= 1.0
    n = 0
    for p in _selected(model, param_filter):
        g = getattr(p, gradient_attr_name, None)
        if g is not None:
            ops.prune_topk_(g, keep_fraction)
            n += 1
    return n


def register_pruning_hooks(model: torch.nn.Module, keep_fraction: float,
                           param_filter: Optional[Callable] = None) -> Iterable:
    """Prune each selected gradient right after autograd accumulated it.  Returns the hook handles
    (``h.remove()`` undoes the registration).  With gradient accumulation over several microbatches the
    hook fires after every microbatch, i.e. the running sum is re-pruned each time."""
    assert 0.0 < keep_fraction <= 1.0

    def hook(param):
        if param.grad is not None:
            ops.prune_topk_(param.grad, keep_fraction)

    return [p.register_post_accumulate_grad_hook(hook) for p in _selected(model, param_filter)]
