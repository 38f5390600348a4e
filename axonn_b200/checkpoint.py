"""Per-tensor-parallel-rank sharded checkpoints.

On-disk layout of the reference (``axonn/checkpoint.py:11-26`` and the
Lightning strategy ``axonn/lightning/axonn_strategy.py:258-293``):
``<folder>/tp_row_R_col_C_depth_D/<name>.pt`` written by data-parallel rank 0
of every tensor-parallel coordinate.  Two reference defects are not carried
over: ``load`` reads the file that ``save`` wrote and returns its content
(the reference looks for ``<prefix>_<name>.pt`` and discards the result,
``checkpoint.py:29-37``), and with pipelining each stage gets its own
``_inter_K`` suffix so stages no longer overwrite one another.
"""

import os

import torch

from . import config


def get_prefix_for_checkpoint() -> str:
    prefix = (
        f"tp_row_{config.intra_layer_row_parallel_rank}"
        f"_col_{config.intra_layer_column_parallel_rank}"
        f"_depth_{config.intra_layer_depth_parallel_rank}"
    )
    if config.G_inter > 1:
        prefix += f"_inter_{config.inter_layer_parallel_rank}"
    return prefix


def checkpoint_path(checkpoint_folder: str, checkpoint_name: str) -> str:
    return os.path.join(checkpoint_folder, get_prefix_for_checkpoint(), f"{checkpoint_name}.pt")


def save(state, checkpoint_folder, checkpoint_name, overwrite=True):
    """Write ``state`` for this tensor-parallel coordinate (DP rank 0 only).

    The file is written to a temporary name and renamed, so a crash during the
    write never leaves a truncated checkpoint behind."""
    if config.data_parallel_rank != 0:
        return None
    path = checkpoint_path(checkpoint_folder, checkpoint_name)
    os.makedirs(os.path.dirname(path), exist_ok=True)
    if os.path.exists(path) and not overwrite:
        raise ValueError(f"Checkpoint {path} already exists")
    tmp = path + f".tmp.{os.getpid()}"
    torch.save(state, tmp)
    os.replace(tmp, path)
    return path


def load(state, checkpoint_folder, checkpoint_name, map_location="cpu"):
    """Load this coordinate's shard file and return it.

    ``state`` may be ``None`` or a dict; when it is a dict its entries are
    updated in place with the loaded ones (and the dict returned), which keeps
    the reference call shape ``state = load(state, folder, name)`` working."""
    if not os.path.isdir(checkpoint_folder):
        raise FileNotFoundError(f"folder {checkpoint_folder} does not exist")
    path = checkpoint_path(checkpoint_folder, checkpoint_name)
    loaded = torch.load(path, map_location=map_location, weights_only=False)
    if isinstance(state, dict) and isinstance(loaded, dict):
        state.update(loaded)
        return state
    return loaded
