"""Device backend of the package's own symmetric heap (csrc/symm_heap.cu) on one GPU: a group of one rank goes
through allocation (cuMemCreate), export, address reservation, mapping and access rights; the mapped slot is then
ordinary device memory.  (The exchange between several ranks is the same code that the CPU tests run on the
host-memory backend.)"""

import pytest
import torch

from _dist import run_distributed

pytestmark = pytest.mark.gpu


def _one_rank_heap(rank, world):
    import torch.distributed as dist

    from axonn_b200.parallel.heap import BACKEND_CUDA, SymmetricHeap

    heap = SymmetricHeap(dist.group.WORLD, 5 << 20)
    assert heap.backend == BACKEND_CUDA and heap.mapped_slots() == 1
    assert heap.slot_bytes >= 5 << 20 and heap.slot_bytes % (2 << 20) == 0 and heap.base % (2 << 20) == 0
    mem = heap.local
    assert mem.is_cuda and mem.numel() == heap.slot_bytes and mem.data_ptr() == heap.peer_ptrs[0]
    mem.fill_(3)
    words = mem[:4096].view(torch.int32)
    words += 1
    torch.cuda.synchronize()
    assert int(mem[:4096].to(torch.int64).sum()) == 3 * 4096 + 1024        # one byte of every word grew by one
    assert int(mem[-1]) == 3
    del mem, words
    heap.close()
    return True


def test_device_backend_maps_usable_memory():
    assert run_distributed(_one_rank_heap, 1, backend="nccl", timeout=120) == [True]
