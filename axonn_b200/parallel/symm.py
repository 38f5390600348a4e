"""Symmetric (peer-mapped) memory for the fused communication kernels.

Each process group that runs fused kernels gets buffers that every rank of the
group maps at a known address: a rank can then load from / store to its peers'
copies directly over NVLink from inside a kernel, and (when the fabric supports
it) reach all copies at once through an NVSwitch multicast address
(``multimem.*``).  Allocation and handle exchange use
``torch.distributed._symmetric_memory`` (CUDA VMM allocations exchanged over
the process group's store) or, with ``AXONN_SYMM_HEAP=own``, the package's own
VMM heap (``parallel/heap.py`` over ``csrc/symm_heap.cu``); this module adds the per-group buffer cache, the
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
    # the output arena survives a re-initialisation of the grid: it is a property of the process (world group)


def enabled() -> bool:
    """Peer-memory kernels are used on CUDA unless ``AXONN_BACKEND=nccl``."""
    if os.environ.get("AXONN_BACKEND", "fused").lower() == "nccl":
        return False
    return torch.cuda.is_available() and _disabled_reason is None


def own_heap_selected() -> bool:
    """``AXONN_SYMM_HEAP=own`` allocates symmetric buffers with the package's own VMM heap (``parallel/heap.py``)
    instead of ``torch.distributed._symmetric_memory`` (the default, ``torch``)."""
    return os.environ.get("AXONN_SYMM_HEAP", "torch").lower() == "own"


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
        if own_heap_selected():
            # the package's own allocator (parallel/heap.py): VMM allocations mapped into one address range;
            # no signal pads (the kernels keep their flags inside the buffers) and no multicast binding
            from .heap import SymmetricHeap

            self.heap = SymmetricHeap(group, self.nbytes + CANARY_BYTES, dev)
            self._full = self.heap.local[:self.nbytes + CANARY_BYTES]
            self._full.zero_()
            self.handle = None
            self.peer_ptrs = list(self.heap.peer_ptrs)
            self.signal_ptrs = []
            self.multicast_ptr = 0
        else:
            self.heap = None
            self._full = symm_mem.empty(self.nbytes + CANARY_BYTES, dtype=torch.uint8, device=dev)
            self.handle = symm_mem.rendezvous(self._full, group=group)
            self.peer_ptrs = [int(p) for p in self.handle.buffer_ptrs]
            self.signal_ptrs = [int(p) for p in self.handle.signal_pad_ptrs]
            self.multicast_ptr = int(getattr(self.handle, "multicast_ptr", 0) or 0)
        self._full[self.nbytes:].fill_(CANARY_VALUE)
        self.local = self._full[:self.nbytes]
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
        if self.handle is None:
            torch.cuda.current_stream().synchronize()
            self.heap.barrier()
        else:
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


class OutputArena:
    """A peer-mapped address range from which the outputs of the two-shot fused all-reduce are allocated.

    The two-shot all-reduce epilogue of the fused GEMM writes finished values into ``C`` on every rank, so
    ``C`` must be memory that the peers have mapped.  One symmetric allocation of ``nbytes`` is made per
    process (rendezvous over the world group, which therefore has to sit on one NVLink domain); a
    ``torch.cuda.MemPool`` whose segment allocator carves that range (``csrc/arena.cu``) lets PyTorch's
    caching allocator place ordinary tensors in it: ``arena.empty(shape, dtype)`` returns a tensor that lives
    as long as anything references it, like any other.  Ranks need not allocate at equal offsets: every call
    of the kernel announces its own offset to its peers through a mailbox in peer memory."""

    def __init__(self, nbytes: int):
        import ctypes

        from ..ops import _lib

        self.group = dist.group.WORLD
        old = os.environ.get("TORCH_SYMM_MEM_DISABLE_MULTICAST")
        os.environ["TORCH_SYMM_MEM_DISABLE_MULTICAST"] = "1"   # plain peer stores only: no multicast binding needed
        try:
            self.buf = SymmBuffer(self.group, int(nbytes), "output_arena")
        finally:
            if old is None:
                os.environ.pop("TORCH_SYMM_MEM_DISABLE_MULTICAST", None)
            else:
                os.environ["TORCH_SYMM_MEM_DISABLE_MULTICAST"] = old
        self.device = self.buf.local.device
        self.base = self.buf.peer_ptrs[self.buf.rank]
        self.nbytes = self.buf.nbytes
        self.peer_base = list(self.buf.peer_ptrs)            # indexed by world rank
        L = _lib.lib()
        L.axb_arena_stat.restype = ctypes.c_ulonglong
        rc = L.axb_arena_register(ctypes.c_int(self.device.index), ctypes.c_void_p(self.base),
                                  ctypes.c_ulonglong(self.nbytes))
        if rc != 0:
            raise RuntimeError("axb_arena_register failed")
        self._allocator = torch.cuda.memory.CUDAPluggableAllocator(_lib.LIB_PATH, "axb_arena_malloc", "axb_arena_free")
        self.pool = torch.cuda.MemPool(self._allocator.allocator())

    def empty(self, shape, dtype):
        try:
            with torch.cuda.use_mem_pool(self.pool, device=self.device):
                return torch.empty(shape, dtype=dtype, device=self.device)
        except torch.OutOfMemoryError as e:
            raise RuntimeError(
                f"the peer-mapped output arena ({self.nbytes / 2**30:.1f} GiB, {self.stat(0) / 2**30:.1f} GiB handed to "
                f"the caching allocator) cannot hold another {tuple(shape)} {dtype} tensor; raise "
                f"AXONN_SYMM_ARENA_GB, or set AXONN_TWO_SHOT=0 to keep all-reduce outputs in ordinary memory") from e

    def offset(self, t) -> int:
        off = t.data_ptr() - self.base
        if not (0 <= off and off + t.numel() * t.element_size() <= self.nbytes):
            raise RuntimeError("tensor does not lie in the output arena")
        return off

    def peer_bases(self, group):
        """Arena base addresses of the ranks of ``group`` (in group order) as mapped in this process."""
        return [self.peer_base[r] for r in dist.get_process_group_ranks(group)]

    def stat(self, what: int) -> int:
        from ..ops import _lib
        import ctypes

        return int(_lib.lib().axb_arena_stat(ctypes.c_int(self.device.index), ctypes.c_int(what)))


_arena: Optional[OutputArena] = None
_arena_tried = False


def output_arena() -> Optional[OutputArena]:
    return _arena


def create_output_arena(nbytes: Optional[int] = None) -> Optional[OutputArena]:
    """Create the process-wide output arena (collective over the world group; ``axonn.init`` calls it when the
    grid has row or column tensor parallelism).  Size: ``nbytes``, else ``AXONN_SYMM_ARENA_GB``, else 40 % of
    the device's memory.  Returns None - and the fused all-reduce stays one-shot, with outputs in ordinary
    memory - when ``AXONN_TWO_SHOT=0``, when the world does not share one peer-memory domain, or when the
    allocation fails on any rank."""
    global _arena, _arena_tried
    if _arena is not None or _arena_tried:
        return _arena
    _arena_tried = True
    if not enabled() or os.environ.get("AXONN_TWO_SHOT", "1") == "0":
        return None
    world = dist.get_world_size()
    if world < 2 or world > 8:
        return None
    from . import fused

    if not fused._peer_capable(dist.group.WORLD):
        return None
    if nbytes is None:
        gb = os.environ.get("AXONN_SYMM_ARENA_GB")
        total = torch.cuda.get_device_properties(torch.cuda.current_device()).total_memory
        nbytes = int(float(gb) * 2**30) if gb else int(total * 0.4)
    nbytes = (int(nbytes) + (1 << 21) - 1) // (1 << 21) * (1 << 21)
    ok, arena = True, None
    try:
        arena = OutputArena(nbytes)
    except Exception as e:  # noqa: BLE001
        ok = False
        reason = str(e)
    flag = torch.tensor([1 if ok else 0], dtype=torch.int32, device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if not bool(flag.item()):
        if dist.get_rank() == 0:
            print(f"axonn_b200: output arena unavailable ({reason if not ok else 'a peer failed'}); "
                  f"fused all-reduce stays one-shot", flush=True)
        return None
    _arena = arena
    return _arena


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
