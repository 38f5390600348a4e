"""Global runtime: ``init``, ``create_dataloader``, timers.

Public contract of the reference's ``axonn/axonn.py:13-127`` — module globals
``comm_handle``, ``config``, ``is_initialized`` and the functions ``init``,
``create_dataloader``, ``get_timers`` — kept verbatim so that
``from axonn_b200 import axonn as ax; ax.init(...)`` is a drop-in for
``from axonn import axonn as ax``.
"""

from typing import Optional

import torch

from . import config
from .communication import communication_handle
from .timers import Timers, _NullTimers

is_initialized = False
comm_handle: Optional[communication_handle] = None
enable_timers = False
timers: Optional[Timers] = None
# compute dtype of the engines/optimizer (bf16 on B200 unless told otherwise)
computation_dtype = torch.bfloat16


def init(
    G_inter: int,
    G_data: int,
    G_intra_r: int = 1,
    G_intra_c: int = 1,
    G_intra_d: int = 1,
    gpus_per_node: Optional[int] = None,
    enable_internal_timers: bool = False,
) -> None:
    """Build the 4-D (inter x data x row/col/depth) process grid.

    Arguments mirror ``axonn/axonn.py:21-29``.  The product of the five grid
    sizes must equal the world size.  On GPUs this also binds the CUDA device
    (``world_rank % gpus_per_node``) and, lazily on first use, the symmetric
    peer-memory heap used by the fused communication kernels.
    """
    global comm_handle, is_initialized, enable_timers, timers
    comm_handle = communication_handle(
        G_inter, G_data, G_intra_r, G_intra_c, G_intra_d, gpus_per_node=gpus_per_node
    )
    config.G_inter = G_inter
    config.G_data = G_data
    config.G_intra = comm_handle.G_intra
    config.G_intra_r = G_intra_r
    config.G_intra_c = G_intra_c
    config.G_intra_d = G_intra_d
    config.inter_layer_parallel_rank = comm_handle.inter_layer_parallel_rank
    config.data_parallel_rank = comm_handle.data_parallel_rank
    config.intra_layer_parallel_rank = comm_handle.intra_layer_parallel_rank
    config.intra_layer_depth_parallel_rank = comm_handle.intra_layer_depth_parallel_rank
    config.intra_layer_row_parallel_rank = comm_handle.intra_layer_row_parallel_rank
    config.intra_layer_column_parallel_rank = comm_handle.intra_layer_column_parallel_rank
    config.device = "cuda" if comm_handle.use_cuda else "cpu"
    is_initialized = True
    enable_timers = enable_internal_timers
    timers = Timers(use_cuda=comm_handle.use_cuda) if enable_internal_timers else _NullTimers()
    # drop per-grid caches of earlier grids (tests re-initialise)
    from .intra_layer import overlap_communication as _oc

    _oc.reset_state()
    from .parallel import symm as _symm

    _symm.reset()
    from .parallel import fused as _fused

    _fused.reset()
    from .parallel import moe_kernels as _mk

    _mk.reset()
    if comm_handle.use_cuda and G_intra_r * G_intra_c > 1:
        # row / column tensor parallelism all-reduces activations inside the GEMM kernels: their outputs live in
        # a peer-mapped arena so that the owner of a tile can store the finished values on every rank
        _symm.create_output_arena()
    elif comm_handle.use_cuda and G_intra_d * G_data > 1:
        # depth / data parallelism only: a small arena serves the stand-alone peer-memory collectives
        # (all-gather, reduce-scatter, row all-to-all of tensors that do not go through a fused GEMM)
        import os

        _symm.create_output_arena(None if os.environ.get("AXONN_SYMM_ARENA_GB") else 2 << 30)


def finalize() -> None:
    """Forget the grid (process groups are left to torch.distributed)."""
    global comm_handle, is_initialized, timers
    comm_handle = None
    is_initialized = False
    timers = None
    config.reset()


def create_dataloader(
    dataset: torch.utils.data.Dataset,
    global_batch_size: int,
    micro_batch_size: int = 1,
    num_workers: int = 0,
    *args,
    **kwargs,
) -> torch.utils.data.DataLoader:
    """Per-rank loader: data is split over ``G_data x G_intra_d`` replicas
    (depth ranks see different samples, like FSDP); the batch size is the
    per-replica batch when pipelining and the microbatch otherwise
    (reference ``axonn/axonn.py:70-121``).  The ``DistributedSampler`` shuffles
    per epoch by default, as upstream; pass ``shuffle=False`` for a fixed order."""
    assert is_initialized, "call init() first"
    replicas = config.G_data * config.G_intra_d
    if global_batch_size % (config.G_data * micro_batch_size) != 0:
        raise ValueError("global_batch_size must be divisible by G_data * micro_batch_size")
    config.micro_batch_size = micro_batch_size
    config.global_batch_size = global_batch_size
    config.batch_size = global_batch_size
    config.batch_size_per_gpu = global_batch_size // replicas
    sampler = torch.utils.data.distributed.DistributedSampler(
        dataset,
        num_replicas=replicas,
        rank=config.G_intra_d * config.data_parallel_rank + config.intra_layer_depth_parallel_rank,
        shuffle=kwargs.pop("shuffle", True),   # the sampler's own default, as in the reference
    )
    bs = config.batch_size_per_gpu if config.G_inter > 1 else micro_batch_size
    kwargs.setdefault("pin_memory", torch.cuda.is_available())
    return torch.utils.data.DataLoader(
        dataset=dataset,
        batch_size=bs,
        shuffle=False,
        num_workers=num_workers,
        sampler=sampler,
        drop_last=True,
        *args,
        **kwargs,
    )


def get_timers() -> Timers:
    """The timers created by ``init(enable_internal_timers=True)`` (a no-op object otherwise)."""
    global timers
    if timers is None:
        timers = _NullTimers()
    return timers
