"""Symmetric (peer-mapped) memory for the fused communication kernels.

Each process group that runs fused kernels gets buffers that every rank of the
group maps at a known address: a rank can then load from / store to its peers'
copies directly over NVLink from inside a kernel, and (when the fabric supports
it) reach all copies at once through an NVSwitch multicast address
(``multimem.*``).  Allocation and handle exchange use
``torch.distributed._symmetric_memory`` (CUDA VMM allocations exchanged over
the process group's store); this module adds the per-group buffer cache, the
peer-pointer tables that kernels take, and monotonically increasing epochs for
the signal pads so that a stale flag can never satisfy a wait.

This is the counterpart of the process-group construction in the reference's
``axonn/communication.py:124-236``, which has no peer-memory path.
"""

import os
import weakref
from typing import Dict, Optional, Tuple

import torch
import torch.distributed as dist

CANARY_BYTES = 256
CANARY_VALUE = 0xA5
_buffers: Dict[Tuple[str, str], "SymmBuffer"] = {}
_all_buffers = []   # weak references to every live SymmBuffer, for verify_canaries()
_disabled_reason: Optional[str] = None


def reset():
    _buffers.clear()


def enabled() -> bool:
    """Peer-memory kernels are used on CUDA unless ``AXONN_BACKEND=nccl``."""
    if os.environ.get("AXONN_BACKEND", "fused").lower() == "nccl":
        return False
    return torch.cuda.is_available() and _disabled_reason is None


def disable(reason: str):
    global _disabled_reason
    _disabled_reason = reason


class SymmBuffer:
    """One symmetric allocation of ``nbytes`` on every rank of ``group``."""

    def __init__(self, group, nbytes: int, tag: str):
        import torch.distributed._symmetric_memory as symm_mem

        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.nbytes = int(nbytes)
        dev = torch.device("cuda", torch.cuda.current_device())
        # CANARY_BYTES guard bytes follow the usable range; kernels never address them, so a changed guard
        # byte means that a kernel (of this rank or of a peer) wrote past the end of the buffer
        self._full = symm_mem.empty(self.nbytes + CANARY_BYTES, dtype=torch.uint8, device=dev)
        self._full[self.nbytes:].fill_(CANARY_VALUE)
        self.local = self._full[:self.nbytes]
        self.handle = symm_mem.rendezvous(self._full, group=group)
        self.peer_ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.signal_ptrs = [int(p) for p in self.handle.signal_pad_ptrs]
        self.multicast_ptr = int(getattr(self.handle, "multicast_ptr", 0) or 0)
        self.ptr_table = torch.tensor(self.peer_ptrs, dtype=torch.int64, device=dev)
        self.signal_table = torch.tensor(self.signal_ptrs, dtype=torch.int64, device=dev)
        self.epoch = 0
        self.tag = tag
        _all_buffers.append(weakref.ref(self))

    def view(self, dtype, numel, offset_bytes=0):
        es = torch.empty((), dtype=dtype).element_size()
        return self.local[offset_bytes:offset_bytes + numel * es].view(dtype)

    def next_epoch(self) -> int:
        self.epoch += 1
        return self.epoch

    def barrier(self):
        self.handle.barrier()

    def canary_intact(self) -> bool:
        """True when the guard bytes behind the buffer still hold their pattern (synchronises the device)."""
        return bool((self._full[self.nbytes:] == CANARY_VALUE).all().item())


def get_buffer(group, nbytes: int, tag: str) -> SymmBuffer:
    """Cached symmetric buffer of at least ``nbytes`` for (group, tag); grows by
    reallocation (collective: every rank of the group must call in step)."""
    key = (str(id(group)), tag)
    buf = _buffers.get(key)
    if buf is None or buf.nbytes < nbytes:
        size = max(int(nbytes), 1 << 20)
        size = (size + (1 << 21) - 1) // (1 << 21) * (1 << 21)
        buf = SymmBuffer(group, size, tag)
        _buffers[key] = buf
    return buf


def debug_bounds_enabled() -> bool:
    return os.environ.get("AXONN_DEBUG_BOUNDS", "0") not in ("", "0")


def verify_canaries():
    """Check the guard bytes of every live symmetric buffer; raises ``RuntimeError`` naming the buffer whose
    guard was overwritten.  Meant to run once per step under ``AXONN_DEBUG_BOUNDS=1`` (it synchronises)."""
    live = []
    for ref in _all_buffers:
        buf = ref()
        if buf is None:
            continue
        live.append(ref)
        if not buf.canary_intact():
            raise RuntimeError(f"symmetric buffer '{buf.tag}' ({buf.nbytes} bytes, group rank {buf.rank}): guard bytes "
                               f"behind the buffer were overwritten - a kernel wrote out of bounds")
    _all_buffers[:] = live
    return len(live)
