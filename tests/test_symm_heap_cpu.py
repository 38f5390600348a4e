"""The package's own symmetric heap (csrc/symm_heap.cu + parallel/heap.py) on CPU ranks: the host-memory backend
runs the same create / export / descriptor exchange / attach sequence as the device backend, with shared pages
in the place of peer-mapped device memory."""

import shutil

import pytest
import torch

from _dist import run_distributed
from axonn_b200.ops import _lib

# the heap is native code: needs the built library, or nvcc to build it on first use
pytestmark = pytest.mark.skipif(not (_lib.available() or shutil.which("nvcc")), reason="native library not built")


def _heap_roundtrip(rank, world):
    import torch.distributed as dist

    from axonn_b200 import axonn as ax
    from axonn_b200.parallel.heap import SymmetricHeap

    ax.init(G_inter=1, G_data=world)
    group = dist.group.WORLD
    heap = SymmetricHeap(group, 3 << 20, device="cpu")            # 3 MiB asked, slots are whole 2 MiB pages
    assert heap.slot_bytes == 4 << 20 and heap.mapped_slots() == world
    assert heap.peer_ptrs == [heap.base + p * heap.slot_bytes for p in range(world)]
    mine = heap.local
    assert mine.numel() == heap.slot_bytes and int(mine.max()) == 0   # fresh pages
    mine[:1024] = rank + 1
    heap.barrier()
    # every rank sees every rank's pattern through its own mapping of that rank's slot
    seen = [int(heap.bytes_of(p)[:1024].to(torch.int64).sum()) for p in range(world)]
    assert seen == [1024 * (p + 1) for p in range(world)], seen
    # a store into the next rank's slot arrives in that rank's own memory
    nxt = (rank + 1) % world
    heap.bytes_of(nxt)[4096 + rank] = 200 + rank
    heap.barrier()
    prev = (rank - 1) % world
    assert int(mine[4096 + prev]) == 200 + prev
    # typed views of a slot share the bytes
    as_f32 = heap.bytes_of(rank)[8192:8192 + 64].view(torch.float32)
    as_f32.fill_(1.5)
    heap.barrier()
    assert float(heap.bytes_of(rank)[8192:8192 + 64].view(torch.float32).sum()) == 24.0
    heap.barrier()
    heap.close()
    return True


@pytest.mark.parametrize("world", [1, 2, 4])
def test_host_backend_maps_every_rank_at_the_same_offsets(world):
    assert all(run_distributed(_heap_roundtrip, world))


def _heap_second_group(rank, world):
    """Two heaps on different groups at once (a pair group and the world), as the fused kernels hold them."""
    import torch.distributed as dist

    from axonn_b200 import axonn as ax
    from axonn_b200.parallel.heap import SymmetricHeap

    ax.init(G_inter=1, G_data=world // 2, G_intra_r=2)
    pair = ax.comm_handle.outer_intra_layer_parallel_group
    a = SymmetricHeap(pair, 1 << 20, device="cpu")
    b = SymmetricHeap(dist.group.WORLD, 1 << 20, device="cpu")
    me = dist.get_rank(pair)
    a.local[0] = 10 + rank
    b.local[0] = 50 + rank
    a.barrier()
    b.barrier()
    partner = [r for r in dist.get_process_group_ranks(pair) if r != rank][0]
    assert int(a.bytes_of(1 - me)[0]) == 10 + partner
    assert [int(b.bytes_of(p)[0]) for p in range(world)] == [50 + p for p in range(world)]
    b.barrier()
    a.close()
    b.close()
    return True


def test_heaps_of_two_groups_coexist():
    assert all(run_distributed(_heap_second_group, 4))


def test_native_heap_rejects_bad_requests():
    import ctypes

    from axonn_b200.ops import _lib

    if not _lib.available():
        pytest.skip("native library not built")
    L = _lib.lib()
    L.axb_heap_create.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_ulonglong,
                                  ctypes.POINTER(ctypes.c_void_p)]
    L.axb_heap_attach.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int]
    L.axb_heap_fd.argtypes = [ctypes.c_void_p]
    L.axb_heap_destroy.argtypes = [ctypes.c_void_p]
    h = ctypes.c_void_p()
    assert L.axb_heap_create(0, 0, 2, 2, 1 << 20, ctypes.byref(h)) == -1        # rank outside the group
    assert L.axb_heap_create(7, 0, 0, 2, 1 << 20, ctypes.byref(h)) == -1        # unknown backend
    assert L.axb_heap_create(0, 0, 0, 2, 0, ctypes.byref(h)) == -1              # empty allocation
    assert L.axb_heap_create(0, 0, 0, 2, 1 << 20, ctypes.byref(h)) == 0
    fd = L.axb_heap_fd(h)
    assert fd >= 0
    assert L.axb_heap_attach(h, 0, fd) == -1                                     # own slot
    assert L.axb_heap_attach(h, 5, fd) == -1                                     # no such peer
    assert L.axb_heap_attach(h, 1, fd) == 0                                      # (its own pages stand in for a peer's)
    assert L.axb_heap_attach(h, 1, fd) == -1 and b"attached already" in L.axb_last_error()
    assert L.axb_heap_destroy(h) == 0


def _heap_silent_peer(rank, world):
    """Rank 1 connects but never hands over its descriptor: every rank gets a clean error, nobody hangs."""
    import os
    import socket

    import torch.distributed as dist

    from axonn_b200 import axonn as ax
    from axonn_b200.parallel.heap import HeapExchangeError, SymmetricHeap

    os.environ["AXONN_HEAP_TIMEOUT_S"] = "5"
    ax.init(G_inter=1, G_data=world)
    if rank == 1:
        socket.send_fds = lambda sock, buffers, fds: 0          # the message is dropped
    try:
        SymmetricHeap(dist.group.WORLD, 1 << 20, device="cpu")
    except HeapExchangeError as e:
        return str(e)
    return "no error"


def test_descriptor_that_never_arrives_is_a_clean_error_on_every_rank():
    out = run_distributed(_heap_silent_peer, 2)
    assert "descriptor exchange" in out[0] and "malformed descriptor message" in out[0]
    assert "descriptor exchange" in out[1] and "on a peer" in out[1]
