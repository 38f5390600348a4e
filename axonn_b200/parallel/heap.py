"""Symmetric heap of a process group, built on the package's own allocator (``csrc/symm_heap.cu``).

Every rank of the group allocates ``nbytes`` (device memory through the CUDA virtual-memory-management API, or
host memory for CPU ranks), exports the allocation as a file descriptor, and maps all ranks' allocations into
one contiguous address range: slot ``p`` of the range is rank ``p``'s memory, at the same offset on every rank.
A kernel reaches a peer's copy of a buffer at ``base + p * slot_bytes + offset``.

The descriptors travel over abstract unix-domain sockets (``SCM_RIGHTS``); the socket names derive from a token
that the group's first rank draws and broadcasts, so the ranks of a group must be processes of one machine -
the same condition as sharing an NVLink domain on an HGX node.  Every wait on a peer is bounded
(``AXONN_HEAP_TIMEOUT_S``, default 120 s) and ends in ``HeapExchangeError`` on the waiting rank.

This replaces the role that NCCL's internal staging buffers play for the process groups of the reference
(``axonn/communication.py:124-236``); ``parallel/symm.py`` selects it with ``AXONN_SYMM_HEAP=own`` instead of
``torch.distributed._symmetric_memory``.
"""

import ctypes
import os
import socket
import struct
import uuid

import torch
import torch.distributed as dist

from ..ops import _lib

BACKEND_HOST, BACKEND_CUDA = 0, 1


class HeapExchangeError(RuntimeError):
    pass


def _timeout_s() -> float:
    return float(os.environ.get("AXONN_HEAP_TIMEOUT_S", "120"))


class _DeviceRange:
    """Hands a device address range to ``torch.as_tensor`` through the CUDA array interface."""

    def __init__(self, address: int, nbytes: int, owner):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (address, False), "version": 3}
        self._owner = owner


class SymmetricHeap:
    """``nbytes`` on every rank of ``group``, all of them mapped here.  Collective over ``group``."""

    def __init__(self, group, nbytes: int, device=None):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if device is None:
            device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else "cpu"
        self.device = torch.device(device)
        self.backend = BACKEND_CUDA if self.device.type == "cuda" else BACKEND_HOST
        L = _lib.lib()
        L.axb_heap_create.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_ulonglong,
                                      ctypes.POINTER(ctypes.c_void_p)]
        L.axb_heap_fd.argtypes = [ctypes.c_void_p]
        L.axb_heap_attach.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int]
        L.axb_heap_info.argtypes = [ctypes.c_void_p, ctypes.c_int]
        L.axb_heap_info.restype = ctypes.c_ulonglong
        L.axb_heap_destroy.argtypes = [ctypes.c_void_p]
        self._L = L
        self._h = ctypes.c_void_p()
        rc = L.axb_heap_create(self.backend, self.device.index or 0, self.rank, self.world, int(nbytes),
                               ctypes.byref(self._h))
        # every rank learns whether every allocation succeeded before anybody waits for descriptors
        self._agree(rc == 0, "allocation")
        self.base = int(L.axb_heap_info(self._h, 0))
        self.slot_bytes = int(L.axb_heap_info(self._h, 1))
        try:
            self._exchange()
            failure = None
        except (OSError, HeapExchangeError) as e:
            failure = e
        self._agree(failure is None, f"descriptor exchange ({failure})")
        self.peer_ptrs = [self.base + p * self.slot_bytes for p in range(self.world)]

    # ------------------------------------------------------------------------------------------------ set-up
    def _error(self) -> str:
        msg = self._L.axb_last_error()
        return msg.decode() if msg else ""

    def _agree(self, ok: bool, what: str):
        flag = torch.tensor([1 if ok else 0], dtype=torch.int32,
                            device=self.device if dist.get_backend(self.group) == "nccl" else "cpu")
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=self.group)
        if not bool(flag.item()):
            mine = f": {self._error()}" if not ok else " on a peer"
            self.close()
            raise HeapExchangeError(f"symmetric heap: {what} failed{mine}")

    def _exchange(self):
        if self.world == 1:
            return
        token = [uuid.uuid4().hex if self.rank == 0 else None]
        dist.broadcast_object_list(token, src=dist.get_global_rank(self.group, 0), group=self.group)
        name = lambda r: f"\0axonn_b200_heap_{token[0]}_{r}"  # noqa: E731  (abstract namespace: no file to clean up)
        listener = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
        try:
            listener.bind(name(self.rank))
            listener.listen(self.world)
            listener.settimeout(_timeout_s())
            dist.barrier(group=self.group)      # every listener exists; connects below cannot be refused
            fd = int(self._L.axb_heap_fd(self._h))
            for peer in range(self.world):
                if peer == self.rank:
                    continue
                with socket.socket(socket.AF_UNIX, socket.SOCK_STREAM) as c:
                    c.settimeout(_timeout_s())
                    c.connect(name(peer))
                    socket.send_fds(c, [struct.pack("i", self.rank)], [fd])
            for _ in range(self.world - 1):
                try:
                    conn, _addr = listener.accept()
                except socket.timeout as e:
                    raise HeapExchangeError("a peer never sent the descriptor of its allocation") from e
                with conn:
                    conn.settimeout(_timeout_s())
                    msg, fds, _flags, _a = socket.recv_fds(conn, 4, 1)
                if len(msg) != 4 or len(fds) != 1:
                    raise HeapExchangeError("malformed descriptor message")
                peer = struct.unpack("i", msg)[0]
                rc = self._L.axb_heap_attach(self._h, peer, fds[0])
                os.close(fds[0])
                if rc != 0:
                    raise HeapExchangeError(self._error())
        finally:
            listener.close()

    # ------------------------------------------------------------------------------------------------ access
    def bytes_of(self, peer: int) -> torch.Tensor:
        """Rank ``peer``'s slot as a ``uint8`` tensor (``peer == self.rank``: this rank's own memory)."""
        address = self.peer_ptrs[peer]
        if self.backend == BACKEND_CUDA:
            return torch.as_tensor(_DeviceRange(address, self.slot_bytes, self), device=self.device)
        raw = (ctypes.c_ubyte * self.slot_bytes).from_address(address)
        t = torch.frombuffer(raw, dtype=torch.uint8)
        t._axonn_heap = self     # the mapping must outlive the view
        return t

    @property
    def local(self) -> torch.Tensor:
        return self.bytes_of(self.rank)

    def mapped_slots(self) -> int:
        return int(self._L.axb_heap_info(self._h, 2))

    def barrier(self):
        dist.barrier(group=self.group)

    def close(self):
        """Unmap and free.  Collective in effect: the caller makes sure no rank still uses the memory."""
        if self._h:
            self._L.axb_heap_destroy(self._h)
            self._h = ctypes.c_void_p()
