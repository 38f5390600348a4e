"""``AxonnStrategy``: run Lightning Fabric programs on the 4-D grid.

Feature parity with the reference's ``axonn/lightning/axonn_strategy.py:59-333``:
the strategy derives ``G_data = world / (r*c*d)`` and calls ``init(G_inter=1)``,
builds modules inside ``auto_parallelize()``, optionally wraps ``forward`` and
``backward`` in ``optimize_communication`` (with reverse-order all-gather
prefetch for backward), synchronises gradients with ``mean=True`` after
backward, honours ``no_backward_sync`` through ``no_grad_sync()``, clips with
the tensor-parallel aware ``clip_grad_norm_`` and stores checkpoints under
``<dir>/tp_row_R_col_C_depth_D/<file>`` written by data-parallel rank 0.

The behaviour lives in ``AxonnStrategyCore`` which has no Lightning
dependency; when ``lightning`` is importable ``AxonnStrategy`` additionally
derives from ``lightning.fabric.strategies.ParallelStrategy`` and plugs the
core into Fabric's hooks.  Without Lightning the same class can be driven
directly (``setup_environment`` / ``setup_module`` / ``backward`` / ...), which
is how it is tested on CPU ranks.
"""

import os
import types
from contextlib import nullcontext
from datetime import timedelta
from typing import Any, Dict, Optional

import torch
import torch.distributed as dist

from .. import axonn as ax
from ..checkpoint import get_prefix_for_checkpoint
from ..intra_layer import (
    auto_parallelize,
    clip_grad_norm_,
    no_grad_sync,
    optimize_communication,
    overlap_all_gathers_for_checkpointed_forward,
    sync_gradients,
)

try:  # pragma: no cover - exercised only where lightning is installed
    from lightning.fabric.strategies.parallel import ParallelStrategy as _FabricBase
    from lightning.fabric.strategies.strategy import _BackwardSyncControl as _SyncBase

    LIGHTNING_AVAILABLE = True
except Exception:  # lightning absent: stand-alone mode
    _FabricBase = object
    _SyncBase = object
    LIGHTNING_AVAILABLE = False


class _NoSyncControl(_SyncBase):
    def no_backward_sync(self, module, enabled: bool = True):
        return no_grad_sync() if enabled else nullcontext()


class AxonnStrategyCore:
    """Grid bring-up and training hooks, independent of Lightning."""

    def _core_init(self, G_intra_r=1, G_intra_c=1, G_intra_d=1, overlap_communication=False, enable_timers=False,
                   activation_checkpointing=None, process_group_backend=None, timeout=None):
        self.G_intra_r, self.G_intra_c, self.G_intra_d = G_intra_r, G_intra_c, G_intra_d
        self.G_data = None
        self.overlap_communication = overlap_communication
        self.enable_timers = enable_timers
        self.activation_checkpointing = activation_checkpointing
        self._process_group_backend = process_group_backend
        self._timeout = timeout or timedelta(minutes=30)
        self._backward_sync_control = _NoSyncControl()

    # ---- distributed bring-up
    def init_grid(self):
        tp = self.G_intra_r * self.G_intra_c * self.G_intra_d
        world = dist.get_world_size()
        if world % tp:
            raise ValueError(f"world size {world} is not divisible by G_intra_r*G_intra_c*G_intra_d = {tp}")
        self.G_data = world // tp
        ax.init(G_inter=1, G_data=self.G_data, G_intra_r=self.G_intra_r, G_intra_c=self.G_intra_c,
                G_intra_d=self.G_intra_d, enable_internal_timers=self.enable_timers)

    @property
    def distributed_sampler_kwargs(self) -> Dict[str, Any]:
        # easy-mode layers take a different batch shard on every rank
        return {"num_replicas": dist.get_world_size(), "rank": dist.get_rank()}

    # ---- module construction
    def module_sharded_context(self):
        return auto_parallelize()

    def module_init_context(self, empty_init: Optional[bool] = None):
        return self.module_sharded_context()

    def setup_module(self, module):
        if self.overlap_communication and not hasattr(module, "_axonn_plain_forward"):
            module._axonn_plain_forward = module.forward

            def forward(self_, *args, **kwargs):
                with optimize_communication(True, True, False, True, self_):
                    return self_._axonn_plain_forward(*args, **kwargs)

            module.forward = types.MethodType(forward, module)
        if self.activation_checkpointing:
            self._wrap_checkpointed(module)
        return module

    def _wrap_checkpointed(self, module):
        from torch.utils.checkpoint import checkpoint

        kinds = self.activation_checkpointing
        kinds = tuple(kinds) if isinstance(kinds, (list, tuple)) else (kinds,)
        for child in module.modules():
            if isinstance(child, kinds) and not hasattr(child, "_axonn_unchecked_forward"):
                child._axonn_unchecked_forward = child.forward

                def fwd(self_, *a, **kw):
                    if not torch.is_grad_enabled():
                        return self_._axonn_unchecked_forward(*a, **kw)
                    return checkpoint(self_._axonn_unchecked_forward, *a, use_reentrant=False, **kw)

                child.forward = types.MethodType(fwd, child)

    # ---- training hooks
    def run_backward(self, tensor, module, call_backward):
        """``call_backward()`` performs autograd; wrapped with overlap + gradient sync."""
        if module is None:
            raise ValueError("pass the model: fabric.backward(loss, model=model)")
        if self.overlap_communication:
            with optimize_communication(True, True, False, True, module):
                with overlap_all_gathers_for_checkpointed_forward(list(module.modules())[::-1]):
                    call_backward()
        else:
            call_backward()
        sync_gradients(module, mean=True)

    def clip_parameters(self, parameters, max_norm, norm_type=2.0, error_if_nonfinite=True):
        return clip_grad_norm_(parameters, max_norm, norm_type, error_if_nonfinite)

    def check_device_status(self):
        """Raise ``AxonnCommTimeout`` if a fused kernel reported an expired device-side wait since the last
        check.  Call it where the training loop already synchronises with the device (after reading the
        loss); ``clip_parameters(..., error_if_nonfinite=True)`` does it as part of its own readback."""
        if torch.cuda.is_available():
            from ..ops import _lib

            _lib.check_status()

    def no_backward_sync(self, module=None, enabled: bool = True):
        return self._backward_sync_control.no_backward_sync(module, enabled)

    @property
    def process_group_backend(self):
        """The backend given at construction (``None``: chosen from the device when the process group is created;
        reference ``axonn/lightning/axonn_strategy.py:116-118``)."""
        return self._process_group_backend

    def get_timers(self):
        assert self.enable_timers, "create the strategy with enable_timers=True"
        return ax.get_timers()

    # ---- checkpoints: <dir>/<tp prefix>/<file>, written by data-parallel rank 0
    @staticmethod
    def sharded_path(path) -> str:
        directory, filename = os.path.split(str(path))
        return os.path.join(directory, get_prefix_for_checkpoint(), filename)

    def save_state(self, path, state: Dict[str, Any]):
        if ax.config.data_parallel_rank != 0:
            return None
        target = self.sharded_path(path)
        os.makedirs(os.path.dirname(target), exist_ok=True)
        plain = {k: (v.state_dict() if hasattr(v, "state_dict") else v) for k, v in state.items()}
        tmp = target + f".tmp.{os.getpid()}"
        torch.save(plain, tmp)
        os.replace(tmp, target)
        return target

    def load_state(self, path, state: Optional[Dict[str, Any]] = None, strict: bool = True):
        loaded = torch.load(self.sharded_path(path), map_location="cpu", weights_only=False)
        if state is None:
            return loaded
        rest = {}
        for k, v in loaded.items():
            obj = state.get(k)
            if isinstance(obj, torch.nn.Module):
                obj.load_state_dict(v, strict=strict)
            elif hasattr(obj, "load_state_dict"):
                obj.load_state_dict(v)
            else:
                state[k] = v
                rest[k] = v
        return rest


if LIGHTNING_AVAILABLE:  # pragma: no cover

    class AxonnStrategy(AxonnStrategyCore, _FabricBase):
        def __init__(self, accelerator=None, parallel_devices=None, cluster_environment=None, checkpoint_io=None,
                     precision=None, process_group_backend=None, timeout=None, G_intra_r=1, G_intra_c=1,
                     G_intra_d=1, overlap_communication=False, enable_timers=False, activation_checkpointing=None,
                     activation_checkpointing_policy=None):
            _FabricBase.__init__(self, accelerator=accelerator, parallel_devices=parallel_devices,
                                 cluster_environment=cluster_environment, checkpoint_io=checkpoint_io,
                                 precision=precision)
            self._core_init(G_intra_r, G_intra_c, G_intra_d, overlap_communication, enable_timers,
                            activation_checkpointing, process_group_backend, timeout)
            self._num_nodes = 1

        @property
        def root_device(self):
            return self.parallel_devices[self.local_rank]

        @property
        def num_nodes(self):
            return self._num_nodes

        @num_nodes.setter
        def num_nodes(self, n):
            self._num_nodes = n

        @property
        def num_processes(self):
            return len(self.parallel_devices) if self.parallel_devices is not None else 0

        def _configure_launcher(self):
            from lightning.fabric.strategies.launchers.subprocess_script import _SubprocessScriptLauncher

            self._launcher = _SubprocessScriptLauncher(self.cluster_environment, self.num_processes, self.num_nodes)

        def setup_environment(self):
            super().setup_environment()
            from lightning.fabric.utilities.distributed import (
                _get_default_process_group_backend_for_device,
                _init_dist_connection,
            )
            from lightning.fabric.utilities.rank_zero import rank_zero_only

            env = self.cluster_environment
            env.set_global_rank(self.node_rank * self.num_processes + self.local_rank)
            env.set_world_size(self.num_nodes * self.num_processes)
            rank_zero_only.rank = self.global_rank
            backend = self._process_group_backend or _get_default_process_group_backend_for_device(self.root_device)
            _init_dist_connection(env, backend, timeout=self._timeout)
            self.init_grid()

        def module_to_device(self, module):
            module.to(self.root_device)

        def all_reduce(self, tensor, group=None, reduce_op="mean"):
            from lightning.fabric.utilities.distributed import _sync_ddp_if_available

            return _sync_ddp_if_available(tensor, group, reduce_op=reduce_op) if torch.is_tensor(tensor) else tensor

        def barrier(self, *args, **kwargs):
            if dist.is_initialized():
                dist.barrier()

        def broadcast(self, obj, src=0):
            if not dist.is_initialized():
                return obj
            box = [obj]
            dist.broadcast_object_list(box, src)
            return box[0]

        def backward(self, tensor, module, *args, **kwargs):
            self.run_backward(tensor, module, lambda: _FabricBase.backward(self, tensor, module, *args, **kwargs))

        def clip_gradients_norm(self, module, optimizer, max_norm, norm_type=2.0, error_if_nonfinite=True):
            self.precision.unscale_gradients(optimizer)
            return self.clip_parameters(self.precision.main_params(optimizer), max_norm, norm_type,
                                        error_if_nonfinite)

        def save_checkpoint(self, path, state, storage_options=None, filter=None):
            if ax.config.data_parallel_rank == 0:
                state = self._convert_stateful_objects_in_state(state, filter=(filter or {}))
                self.checkpoint_io.save_checkpoint(checkpoint=state, path=self.sharded_path(path),
                                                   storage_options=storage_options)

        def load_checkpoint(self, path, state=None, strict=True):
            return super().load_checkpoint(self.sharded_path(path), state, strict)

        @classmethod
        def register_strategies(cls, strategy_registry):
            pass

else:

    class AxonnStrategy(AxonnStrategyCore):
        """Stand-alone form used when Lightning is not installed.

        Drive it like Fabric would::

            s = AxonnStrategy(G_intra_r=2, overlap_communication=True)
            s.setup_environment()                 # torch.distributed must be initialised
            with s.module_init_context():
                model = build_model()             # nn.Linear -> tensor-parallel Linear
            model = s.setup_module(model)
            s.backward(loss, model)               # autograd + gradient sync
            s.clip_gradients_norm(model, optimizer, 1.0)
            s.save_checkpoint("ckpt/step.pt", {"model": model, "optimizer": optimizer})
        """

        def __init__(self, G_intra_r=1, G_intra_c=1, G_intra_d=1, overlap_communication=False, enable_timers=False,
                     activation_checkpointing=None, process_group_backend=None, timeout=None, **_ignored):
            self._core_init(G_intra_r, G_intra_c, G_intra_d, overlap_communication, enable_timers,
                            activation_checkpointing, process_group_backend, timeout)

        def setup_environment(self):
            if not dist.is_initialized():
                raise RuntimeError("initialise torch.distributed (e.g. torchrun) before setup_environment()")
            self.init_grid()

        def backward(self, tensor, module, *args, **kwargs):
            self.run_backward(tensor, module, lambda: tensor.backward(*args, **kwargs))

        def clip_gradients_norm(self, module, optimizer, max_norm, norm_type=2.0, error_if_nonfinite=True):
            params = [p for g in optimizer.param_groups for p in g["params"]]
            return self.clip_parameters(params, max_norm, norm_type, error_if_nonfinite)

        def save_checkpoint(self, path, state, storage_options=None, filter=None):
            return self.save_state(path, state)

        def load_checkpoint(self, path, state=None, strict=True):
            return self.load_state(path, state, strict)
