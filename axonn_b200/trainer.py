"""Training-step driver for models without pipelining (``G_inter == 1``).

``Trainer.train_step(tokens, targets)`` is the call a user makes once per
optimizer step.  It takes this rank's batch (host tensors, ideally pinned),
copies it to the GPU, runs forward/backward over microbatches inside
``optimize_communication`` with gradient synchronisation deferred to the last
microbatch, optionally prunes gradients (top-k by magnitude), synchronises and
clips them, steps the optimizer and returns the mean loss as a Python float.

It packages the loop the reference leaves to user scripts and to its Lightning
strategy (``axonn/lightning/axonn_strategy.py:148-164,241-256``).
"""

import os
from typing import Callable, Optional

import torch
import torch.distributed as dist

from . import axonn as ax
from . import ops
from .ops import _lib
from .parallel import symm
from .intra_layer import (clip_grad_norm_, no_grad_sync, optimize_communication,
                          overlap_all_gathers_for_checkpointed_forward, sync_gradients)


class Trainer:
    """One optimizer step per call for models without pipelining: ``train_step(tokens, targets)`` (host tensors in,
    loss as a float out) and ``train_step_device`` (device tensors, loss stays on the device).  Microbatches of
    ``micro_batch_size``, communication overlap, optional top-k gradient pruning (``prune_keep_fraction``),
    gradient synchronisation, clipping at ``clip_grad`` and the optimizer step."""

    def __init__(self, model, optimizer, micro_batch_size: Optional[int] = None, clip_grad: float = 0.0,
                 prune_keep_fraction: Optional[float] = None, overlap: bool = True,
                 loss_fn: Optional[Callable] = None, expert_mode: bool = True,
                 prefetch_all_gather: Optional[bool] = None):
        assert ax.is_initialized
        if ax.config.G_inter != 1:
            raise ValueError("Trainer drives non-pipelined models; use AxoNN_Inter_Layer_Engine for G_inter > 1")
        self.model, self.optimizer = model, optimizer
        self.micro_batch_size = micro_batch_size
        self.clip_grad = clip_grad
        self.prune_keep_fraction = prune_keep_fraction
        self.overlap = overlap
        # depth all-gathers: by default the GEMM kernels gather their weight shards themselves over peer memory
        # while they compute; AXONN_AG_PREFETCH=1 (or prefetch_all_gather=True) prefetches them one layer ahead
        # with the collective library on a side stream instead (also what CPU ranks do)
        if prefetch_all_gather is None:
            prefetch_all_gather = os.environ.get("AXONN_AG_PREFETCH", "0") == "1"
        self.prefetch_all_gather = prefetch_all_gather and overlap
        self.loss_fn = loss_fn
        self.expert_mode = expert_mode
        self.device = ax.comm_handle.device
        self._params = [p for p in model.parameters() if p.requires_grad]
        self._reversed_modules = list(model.modules())[::-1]

    # ------------------------------------------------------------------ pieces
    def _to_device(self, t):
        if t.device == self.device:
            return t
        return t.to(self.device, non_blocking=True)

    def _forward_loss(self, inputs, targets):
        if self.loss_fn is None:
            return self.model(inputs, targets)
        return self.loss_fn(self.model(inputs), targets)

    def forward_backward(self, inputs, targets):
        """Microbatched forward/backward on device tensors; returns the mean loss
        as a 0-d device tensor.  Gradients are left unsynchronised."""
        B = inputs.shape[0]
        mbs = self.micro_batch_size or B
        n_micro = max(1, B // mbs)
        total = None
        for i in range(n_micro):
            x, y = inputs[i * mbs:(i + 1) * mbs], targets[i * mbs:(i + 1) * mbs]
            with optimize_communication(overlap_all_reduce=self.overlap, overlap_reduce_scatter=self.overlap,
                                        cache_weights=False, overlap_all_gather=self.prefetch_all_gather,
                                        model_object_for_overlapping_allgathers=self.model):
                loss = self._forward_loss(x, y)
                # backward consumes the layers in reverse: prefetch depth all-gathers in that order
                with overlap_all_gathers_for_checkpointed_forward(self._reversed_modules):
                    (loss / n_micro).backward()
            total = loss.detach() if total is None else total + loss.detach()
        return total / n_micro

    def finish_step(self):
        """Prune (optional), synchronise, clip (optional) and apply gradients."""
        if self.prune_keep_fraction is not None:
            for p in self._params:
                if p.grad is not None and p.grad.numel() >= 1024:
                    ops.prune_topk_(p.grad, self.prune_keep_fraction)
        sync_gradients(self.model, mean=True, expert_mode=self.expert_mode)
        if self.clip_grad and self.clip_grad > 0:
            clip_grad_norm_(self._params, self.clip_grad)
        self.optimizer.step()
        self.optimizer.zero_grad(set_to_none=True)

    # ------------------------------------------------------------------ public step
    def train_step_device(self, inputs, targets):
        """One optimizer step on tensors that already live on the device; returns a
        0-d device tensor (no host synchronisation)."""
        self.model.train()
        with no_grad_sync():
            loss = self.forward_backward(inputs, targets)
        self.finish_step()
        return loss

    def train_step(self, inputs, targets) -> float:
        """One optimizer step from host tensors; returns the loss as a float."""
        loss = self.train_step_device(self._to_device(inputs), self._to_device(targets))
        value = float(loss.item())
        _lib.check_status()   # a bounded device-side wait that gave up surfaces here, after the sync above
        if symm.debug_bounds_enabled():
            symm.verify_canaries()
        return value

    # ------------------------------------------------------------------ a whole run, restartable
    def fit(self, batches, steps: int, checkpoint_folder: Optional[str] = None, checkpoint_every: int = 0,
            resume: bool = True, watchdog=None, on_step: Optional[Callable] = None):
        """Run optimizer steps ``first .. steps - 1`` over ``batches`` and return ``{step: loss}``.

        ``batches(step)`` returns the ``(inputs, targets)`` of this rank for a step (a function of the step
        number, so that a restarted run sees the data the first run would have seen).  With ``checkpoint_folder``
        a grid-independent checkpoint is written every ``checkpoint_every`` steps (``checkpoint.save_consolidated``)
        and the name of the newest complete one is recorded in ``<folder>/latest``; with ``resume`` a run that
        finds such a record continues from it - on the same grid or on another one.  ``watchdog`` (a started
        ``parallel.watchdog.Watchdog``) is checked at every step boundary, so a silent peer ends the run with
        ``RankFailure`` instead of a blocked collective.  ``on_step(step, loss)`` is called after every step.

        The reference leaves all of this to the user's script; it has no restart logic."""
        from . import checkpoint

        first = 0
        marker = os.path.join(checkpoint_folder, "latest") if checkpoint_folder else None
        if marker and resume and os.path.exists(marker):
            with open(marker) as f:
                name = f.read().strip()
            first = int(checkpoint.load_consolidated(self.model, self.optimizer, checkpoint_folder, name)["step"])
        losses = {}
        for step in range(first, steps):
            if watchdog is not None:
                watchdog.check()
            inputs, targets = batches(step)
            losses[step] = self.train_step(inputs, targets)
            if on_step is not None:
                on_step(step, losses[step])
            done = step + 1
            if marker and checkpoint_every and done % checkpoint_every == 0:
                name = f"step{done}"
                checkpoint.save_consolidated(self.model, self.optimizer, checkpoint_folder, name, extra={"step": done})
                if dist.is_initialized():
                    dist.barrier()                      # every stage's file is complete before the record moves
                if not dist.is_initialized() or dist.get_rank() == 0:
                    tmp = marker + f".tmp.{os.getpid()}"
                    with open(tmp, "w") as f:
                        f.write(name)
                    os.replace(tmp, marker)
        return losses


def replica_index() -> int:
    """Index of this rank's data shard: ranks that differ only in row/column
    coordinates consume the same samples."""
    c = ax.config
    return c.data_parallel_rank * c.G_intra_d + c.intra_layer_depth_parallel_rank


def num_replicas() -> int:
    """Number of different data shards per step: data-parallel size x depth size."""
    return ax.config.G_data * ax.config.G_intra_d


def all_reduce_max(value: float, device) -> float:
    """Maximum of a host value over all ranks (how multi-GPU timings are reported)."""
    t = torch.tensor([value], dtype=torch.float64, device=device)
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())
