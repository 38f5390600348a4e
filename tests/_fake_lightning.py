"""A stand-in for the part of ``lightning.fabric`` that ``AxonnStrategy`` builds on, for machines without Lightning.

It follows the shapes of the public Lightning Fabric classes (``ParallelStrategy`` with its accelerator /
parallel devices / cluster environment / checkpoint io / precision plugins, ``_BackwardSyncControl``, the
subprocess launcher, the distributed helpers) closely enough that the Fabric-facing subclass of the strategy runs
its own code - hooks, properties, checkpoint paths - on CPU ranks.  It is not Lightning: a test that passes here
shows that the subclass is internally consistent, not that it matches a given Lightning release."""

import sys
import types

import torch
import torch.distributed as dist


class _BackwardSyncControl:
    def no_backward_sync(self, module, enabled=True):
        raise NotImplementedError


class Precision:
    def backward(self, tensor, model, *args, **kwargs):
        tensor.backward(*args, **kwargs)

    def unscale_gradients(self, optimizer):
        return None

    def main_params(self, optimizer):
        for group in optimizer.param_groups:
            yield from group["params"]


class TorchCheckpointIO:
    def save_checkpoint(self, checkpoint, path, storage_options=None):
        import os

        os.makedirs(os.path.dirname(path), exist_ok=True)
        torch.save(checkpoint, path)

    def load_checkpoint(self, path, map_location=None):
        return torch.load(path, map_location=map_location, weights_only=False)


class ClusterEnvironment:
    """Environment of one process started by an external launcher (rank and world size known up front)."""

    def __init__(self, rank, world, main_port):
        self._rank, self._world, self.main_port, self.main_address = rank, world, main_port, "127.0.0.1"

    def local_rank(self):
        return self._rank

    def node_rank(self):
        return 0

    def global_rank(self):
        return self._rank

    def world_size(self):
        return self._world

    def set_global_rank(self, rank):
        self._rank = rank

    def set_world_size(self, n):
        self._world = n


class Strategy:
    def __init__(self, accelerator=None, checkpoint_io=None, precision=None):
        self._accelerator, self._checkpoint_io, self._precision = accelerator, checkpoint_io, precision
        self._launcher = None
        self._backward_sync_control = None

    @property
    def checkpoint_io(self):
        if self._checkpoint_io is None:
            self._checkpoint_io = TorchCheckpointIO()
        return self._checkpoint_io

    @property
    def precision(self):
        if self._precision is None:
            self._precision = Precision()
        return self._precision

    @property
    def launcher(self):
        return self._launcher

    def setup_environment(self):
        self.root_device  # noqa: B018  (the real class sets the accelerator up for this device)

    def backward(self, tensor, module, *args, **kwargs):
        self.precision.backward(tensor, module, *args, **kwargs)

    def _convert_stateful_objects_in_state(self, state, filter):
        out = {}
        for key, obj in state.items():
            out[key] = obj.state_dict() if hasattr(obj, "state_dict") else obj
        return out

    def load_checkpoint(self, path, state=None, strict=True):
        checkpoint = self.checkpoint_io.load_checkpoint(path)
        if not state:
            return checkpoint
        for key, obj in state.items():
            if key not in checkpoint:
                continue
            if isinstance(obj, torch.nn.Module):
                obj.load_state_dict(checkpoint.pop(key), strict=strict)
            elif hasattr(obj, "load_state_dict"):
                obj.load_state_dict(checkpoint.pop(key))
            else:
                state[key] = checkpoint.pop(key)
        return checkpoint


class ParallelStrategy(Strategy):
    def __init__(self, accelerator=None, parallel_devices=None, cluster_environment=None, checkpoint_io=None,
                 precision=None):
        super().__init__(accelerator=accelerator, checkpoint_io=checkpoint_io, precision=precision)
        self.parallel_devices = parallel_devices
        self.cluster_environment = cluster_environment

    @property
    def global_rank(self):
        return self.cluster_environment.global_rank() if self.cluster_environment is not None else 0

    @property
    def local_rank(self):
        return self.cluster_environment.local_rank() if self.cluster_environment is not None else 0

    @property
    def node_rank(self):
        return self.cluster_environment.node_rank() if self.cluster_environment is not None else 0

    @property
    def world_size(self):
        return self.cluster_environment.world_size() if self.cluster_environment is not None else 1


class _SubprocessScriptLauncher:
    def __init__(self, cluster_environment, num_processes, num_nodes):
        self.cluster_environment, self.num_processes, self.num_nodes = cluster_environment, num_processes, num_nodes


def _get_default_process_group_backend_for_device(device):
    return "nccl" if device.type == "cuda" else "gloo"


def _init_dist_connection(cluster_environment, torch_distributed_backend, global_rank=None, world_size=None, **kwargs):
    if dist.is_initialized():
        return
    rank = cluster_environment.global_rank() if global_rank is None else global_rank
    world = cluster_environment.world_size() if world_size is None else world_size
    dist.init_process_group(torch_distributed_backend, rank=rank, world_size=world,
                            init_method=f"tcp://{cluster_environment.main_address}:{cluster_environment.main_port}",
                            **kwargs)


def _sync_ddp_if_available(result, group=None, reduce_op=None):
    if not (dist.is_available() and dist.is_initialized()):
        return result
    mean = isinstance(reduce_op, str) and reduce_op.lower() in ("mean", "avg")
    dist.all_reduce(result, group=group)
    if mean:
        result = result / dist.get_world_size(group)
    return result


class _RankZeroOnly:
    rank = 0


def install():
    """Register the stand-in under the ``lightning.fabric`` module names that the strategy imports."""
    def module(name, **attrs):
        m = types.ModuleType(name)
        m.__dict__.update(attrs)
        sys.modules[name] = m
        return m

    module("lightning")
    module("lightning.fabric")
    module("lightning.fabric.strategies")
    module("lightning.fabric.strategies.parallel", ParallelStrategy=ParallelStrategy)
    module("lightning.fabric.strategies.strategy", _BackwardSyncControl=_BackwardSyncControl, Strategy=Strategy)
    module("lightning.fabric.strategies.launchers")
    module("lightning.fabric.strategies.launchers.subprocess_script", _SubprocessScriptLauncher=_SubprocessScriptLauncher)
    module("lightning.fabric.utilities")
    module("lightning.fabric.utilities.distributed",
           _get_default_process_group_backend_for_device=_get_default_process_group_backend_for_device,
           _init_dist_connection=_init_dist_connection, _sync_ddp_if_available=_sync_ddp_if_available)
    module("lightning.fabric.utilities.rank_zero", rank_zero_only=_RankZeroOnly)
