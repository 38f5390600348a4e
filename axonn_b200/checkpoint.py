"""Per-tensor-parallel-rank sharded checkpoints.

On-disk layout of the reference (``axonn/checkpoint.py:11-26`` and the
Lightning strategy ``axonn/lightning/axonn_strategy.py:258-293``):
``<folder>/tp_row_R_col_C_depth_D/<name>.pt`` written by data-parallel rank 0
of every tensor-parallel coordinate.  Two reference defects are not carried
over: ``load`` reads the file that ``save`` wrote and returns its content
(the reference looks for ``<prefix>_<name>.pt`` and discards the result,
``checkpoint.py:29-37``), and with pipelining each stage gets its own
``_inter_K`` suffix so stages no longer overwrite one another.

Besides the per-coordinate shard files there is a grid-independent form
(:func:`consolidated_state`, :func:`save_consolidated`,
:func:`load_consolidated`): every tensor-parallel parameter and every
optimizer state tensor laid out like one is reassembled to its full shape, so a
run can be resumed on a different ``(G_data, G_intra_r, G_intra_c, G_intra_d)``
grid, e.g. after losing a node.  The reference has only the loading half of this
(``axonn/intra_layer/fully_connected.py:350-400`` accepts a full matrix or a
matching shard) and no optimizer-state resharding.
"""

import os

import torch

from . import config


def get_prefix_for_checkpoint() -> str:
    """``tp_row_R_col_C_depth_D`` of this rank (``_inter_K`` appended when pipelining)."""
    prefix = (
        f"tp_row_{config.intra_layer_row_parallel_rank}"
        f"_col_{config.intra_layer_column_parallel_rank}"
        f"_depth_{config.intra_layer_depth_parallel_rank}"
    )
    if config.G_inter > 1:
        prefix += f"_inter_{config.inter_layer_parallel_rank}"
    return prefix


def checkpoint_path(checkpoint_folder: str, checkpoint_name: str) -> str:
    """``<folder>/<prefix of this rank>/<name>.pt``."""
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


# ----------------------------------------------------------------------------------------------------------
# Writing in the background
# ----------------------------------------------------------------------------------------------------------

class PendingSave:
    """Handle of a checkpoint that is being written by a background thread."""

    def __init__(self, path):
        self.path = path
        self._thread = None
        self._error = None

    def done(self) -> bool:
        return self._thread is None or not self._thread.is_alive()

    def wait(self):
        """Block until the file is in place; re-raises whatever the writer thread raised."""
        if self._thread is not None:
            self._thread.join()
            self._thread = None
        if self._error is not None:
            err, self._error = self._error, None
            raise err
        return self.path


_pending = None


def _snapshot(obj, stream):
    """Copy of ``obj`` (nested dicts / lists / tuples of tensors and plain values) in host memory.  Device tensors
    are copied on ``stream`` into pinned buffers without blocking the host; host tensors are cloned."""
    if torch.is_tensor(obj):
        if obj.is_cuda:
            host = torch.empty(obj.shape, dtype=obj.dtype, device="cpu", pin_memory=True)
            with torch.cuda.stream(stream):
                host.copy_(obj, non_blocking=True)
            obj.record_stream(stream)      # the allocator must not hand the source to someone else before the copy ran
            return host
        return obj.detach().clone()
    if isinstance(obj, dict):
        return type(obj)((k, _snapshot(v, stream)) for k, v in obj.items())
    if isinstance(obj, (list, tuple)):
        return type(obj)(_snapshot(v, stream) for v in obj)
    return obj


def save_async(state, checkpoint_folder, checkpoint_name, overwrite=True):
    """:func:`save` without stopping the training loop for the file write.

    The call returns after a snapshot of ``state`` has been started: device tensors are copied to pinned host
    memory on a side stream that waits for the work already queued on the current stream (so the snapshot holds
    the values as of this call, and later optimizer steps may overwrite the originals at once), host tensors
    are cloned.  A background thread waits for the copies, writes the file under a temporary name and renames it.
    Only one write is in flight: a second call first waits for the previous one.  Returns a :class:`PendingSave`
    (``None`` on ranks that do not write); :func:`wait_for_pending_save` blocks until the file exists - call it
    before the process exits."""
    import threading

    global _pending
    wait_for_pending_save()
    if config.data_parallel_rank != 0:
        return None
    path = checkpoint_path(checkpoint_folder, checkpoint_name)
    os.makedirs(os.path.dirname(path), exist_ok=True)
    if os.path.exists(path) and not overwrite:
        raise ValueError(f"Checkpoint {path} already exists")
    stream = event = None
    if torch.cuda.is_available() and torch.cuda.is_initialized():
        stream = torch.cuda.Stream()
        stream.wait_stream(torch.cuda.current_stream())
    snap = _snapshot(state, stream)
    if stream is not None:
        event = torch.cuda.Event()
        event.record(stream)
    pending = PendingSave(path)

    def write():
        try:
            if event is not None:
                event.synchronize()
            tmp = path + f".tmp.{os.getpid()}"
            torch.save(snap, tmp)
            os.replace(tmp, path)
        except BaseException as e:  # noqa: BLE001  (handed to the caller of wait())
            pending._error = e

    pending._thread = threading.Thread(target=write, name="axonn-checkpoint-writer", daemon=False)
    pending._thread.start()
    _pending = pending
    return pending


def wait_for_pending_save():
    """Block until the checkpoint started by the last :func:`save_async` is on disk (no-op when there is none)."""
    global _pending
    if _pending is not None:
        pending, _pending = _pending, None
        pending.wait()


# ----------------------------------------------------------------------------------------------------------
# Grid-independent checkpoints
# ----------------------------------------------------------------------------------------------------------

_PER_PARAMETER_STATE = ("master", "exp_avg", "exp_avg_sq", "momentum_buffer")


def _sharded_parameters(model):
    """``{parameter name: (module, local name)}`` for every parameter whose owning module knows how to rebuild
    the full tensor (``full_tensor`` / ``shard_tensor``: the tensor-parallel layers, the split-hidden norms, the
    expert-parallel MoE layer).  All other parameters are replicated and stored as they are."""
    out = {}
    for mname, module in model.named_modules():
        if not (hasattr(module, "full_tensor") and hasattr(module, "shard_tensor")):
            continue
        for pname, _ in module.named_parameters(recurse=False):
            out[(mname + "." if mname else "") + pname] = (module, pname)
    return out


def _is_consolidation_writer() -> bool:
    return config.data_parallel_rank == 0 and config.intra_layer_parallel_rank == 0


def _consolidated_path(folder, name):
    stage = f".inter_{config.inter_layer_parallel_rank}" if config.G_inter > 1 else ""
    return os.path.join(folder, f"{name}.full{stage}.pt")


@torch.no_grad()
def consolidated_state(model, optimizer=None, keep=None):
    """Reassemble the model (and optionally the optimizer state) into full, grid-independent tensors.

    Collective: every rank of the job calls it with the same model.  Tensors are gathered one at a time and
    moved to host memory; ranks for which ``keep`` is false (default: all but data-parallel rank 0 /
    tensor-parallel rank 0 of each pipeline stage) drop them at once and get ``None`` back, so at most one
    full tensor is alive on a device at any time.

    The optimizer part is keyed by parameter *name*, not by index: ``{"state": {name: {"step": n, "exp_avg":
    full tensor, ...}}, "param_groups": [hyper-parameters without the parameter lists]}``."""
    keep = _is_consolidation_writer() if keep is None else keep
    sharded = _sharded_parameters(model)
    out_model = {}
    for name, value in model.state_dict().items():
        if name in sharded:
            module, pname = sharded[name]
            value = module.full_tensor(pname, value)
        if keep:
            out_model[name] = value.detach().to("cpu", copy=True)
        del value
    state = {"model": out_model if keep else None}
    if optimizer is not None:
        names = {p: n for n, p in model.named_parameters()}
        opt_state = {}
        for group in optimizer.param_groups:
            for p in group["params"]:
                name, st = names.get(p), optimizer.state.get(p)
                if name is None or not st:
                    continue
                entry = {}
                for key, value in st.items():
                    if torch.is_tensor(value) and key in _PER_PARAMETER_STATE and value.numel() == p.numel():
                        value = value.to(p.device).view_as(p)
                        if name in sharded:
                            module, pname = sharded[name]
                            value = module.full_tensor(pname, value)
                        value = value.detach().to("cpu", copy=True) if keep else None
                    elif torch.is_tensor(value):
                        value = value.detach().to("cpu", copy=True) if keep else None
                    entry[key] = value
                if keep:
                    opt_state[name] = entry
        groups = [{k: v for k, v in g.items() if k != "params"} for g in optimizer.param_groups]
        state["optimizer"] = {"state": opt_state, "param_groups": groups,
                              "steps": getattr(optimizer, "_steps", None)} if keep else None
    return state if keep else None


def save_consolidated(model, optimizer, checkpoint_folder, checkpoint_name, extra=None, overwrite=True):
    """Write ``<folder>/<name>.full.pt`` (``.full.inter_K.pt`` per pipeline stage): one file that any grid can
    load.  Collective; one rank per pipeline stage writes.  ``extra`` (step counters, RNG state, ...) is stored
    under ``"extra"``.  Returns the path on the writing rank, ``None`` elsewhere."""
    state = consolidated_state(model, optimizer)
    if state is None:
        return None
    if extra is not None:
        state["extra"] = extra
    state["grid"] = {k: getattr(config, k) for k in ("G_inter", "G_data", "G_intra_r", "G_intra_c", "G_intra_d")}
    path = _consolidated_path(checkpoint_folder, checkpoint_name)
    os.makedirs(checkpoint_folder, exist_ok=True)
    if os.path.exists(path) and not overwrite:
        raise ValueError(f"Checkpoint {path} already exists")
    tmp = path + f".tmp.{os.getpid()}"
    torch.save(state, tmp)
    os.replace(tmp, path)
    return path


@torch.no_grad()
def load_consolidated(model, optimizer, checkpoint_folder, checkpoint_name, strict=True):
    """Load a file written by :func:`save_consolidated` into a model / optimizer living on *this* grid.

    Every rank reads the file (memory-mapped, so the ranks of a node share the page cache) and keeps its own
    piece of each tensor: the layers' state-dict hooks cut the model tensors, ``shard_tensor`` cuts the
    optimizer's.  No communication.  Returns the ``"extra"`` entry (or ``None``)."""
    path = _consolidated_path(checkpoint_folder, checkpoint_name)
    try:
        state = torch.load(path, map_location="cpu", weights_only=False, mmap=True)
    except (RuntimeError, ValueError):
        state = torch.load(path, map_location="cpu", weights_only=False)
    model.load_state_dict(state["model"], strict=strict)
    saved = state.get("optimizer")
    if optimizer is not None and saved is not None:
        sharded = _sharded_parameters(model)
        names = {p: n for n, p in model.named_parameters()}
        for group, hyper in zip(optimizer.param_groups, saved["param_groups"]):
            group.update(hyper)
            for p in group["params"]:
                entry = saved["state"].get(names.get(p))
                if entry is None:
                    continue
                host_state = hasattr(optimizer, "_host_state")  # CPUAdam: flat fp32 state in pinned host memory
                st = optimizer._host_state(p) if host_state else optimizer.state[p]
                for key, value in entry.items():
                    if torch.is_tensor(value) and key in _PER_PARAMETER_STATE:
                        if names[p] in sharded and value.shape != p.shape:
                            module, pname = sharded[names[p]]
                            value = module.shard_tensor(pname, value)
                        if host_state:
                            st[key].copy_(value.reshape(-1))
                            continue
                        value = value.to(device=p.device, copy=True).contiguous()
                    elif torch.is_tensor(value):
                        value = value.to(device=p.device, copy=True)
                    st[key] = value
        if saved.get("steps") is not None and hasattr(optimizer, "_steps"):
            optimizer._steps = int(saved["steps"])
        if hasattr(optimizer, "_tables"):
            optimizer._tables.clear()  # cached pointer tables name the replaced state tensors
    return state.get("extra")
