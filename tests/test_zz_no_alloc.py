"""The allocation-free pruning entry point (``axb_prune_topk_static``).

It serves programs that manage all device memory themselves and therefore can
neither pass freshly allocated scratch nor let the library allocate: its
workspace is a fixed array inside the library.  The test calls the exported C
symbol directly, twice in a row on different data (the shared scratch keeps the
previous call's contents, so the second call proves it is cleared), and
requires bit-identical results to the workspace-taking entry point.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _call_static(lib, g, k):
    code = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}[g.dtype]   # codes of csrc/axonn_b200.h
    return lib.axb_prune_topk_static(ctypes.c_void_p(g.data_ptr()), ctypes.c_longlong(g.numel()), ctypes.c_int(code),
                                     ctypes.c_longlong(k), ctypes.c_int(g.device.index),
                                     ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))


def test_static_scratch_entry_point_matches_workspace_version():
    from axonn_b200 import ops
    from axonn_b200.ops import _lib

    lib = _lib.lib()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    torch.manual_seed(0)
    for n, dtype in [(1_000_003, torch.bfloat16), (300_000, torch.float32), (1_000_003, torch.bfloat16)]:
        g = torch.randn(n, device=dev).to(dtype) * (1.0 + torch.rand(1, device=dev).item())
        k = max(1, int(round(n * 0.1)))
        want = ops.prune_topk_(g.clone(), 0.1)          # existing entry point (caller-supplied workspace)
        got = g.clone()
        assert _call_static(lib, got, k) == 0, lib.axb_last_error()
        torch.cuda.synchronize()
        assert torch.equal(got, want)
        assert int((got != 0).sum()) >= k


def test_static_entry_point_rejects_oversized_request():
    from axonn_b200.ops import _lib

    lib = _lib.lib()
    g = torch.zeros(8, device="cuda:0")
    st = lib.axb_prune_topk_static(ctypes.c_void_p(g.data_ptr()), ctypes.c_longlong(2 ** 31), ctypes.c_int(2),
                                   ctypes.c_longlong(1), ctypes.c_int(0),
                                   ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert st != 0 and b"exceed" in lib.axb_last_error()


def test_static_entry_point_stays_inside_a_bf16_tensor():
    """A bf16 tensor passed with the header's code for bf16 (0) is pruned as 2-byte elements: the guard
    elements placed directly behind it keep their values."""
    from axonn_b200 import ops
    from axonn_b200.ops import _lib

    lib = _lib.lib()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    torch.manual_seed(1)
    n, guard = 262_144 + 24, 4096
    whole = torch.randn(n + guard, device=dev).to(torch.bfloat16)
    whole[n:] = 7.0
    g = whole[:n]
    want = ops.prune_topk_(g.clone(), 0.25)
    assert _call_static(lib, g, max(1, int(round(n * 0.25)))) == 0, lib.axb_last_error()
    torch.cuda.synchronize()
    assert torch.equal(g, want)
    assert bool((whole[n:] == 7.0).all()), "the entry point wrote behind the tensor"


def test_static_entry_point_requires_the_current_device():
    from axonn_b200.ops import _lib

    lib = _lib.lib()
    g = torch.zeros(64, device="cuda:0")
    torch.cuda.set_device(0)
    st = lib.axb_prune_topk_static(ctypes.c_void_p(g.data_ptr()), ctypes.c_longlong(64), ctypes.c_int(2),
                                   ctypes.c_longlong(8), ctypes.c_int(1),
                                   ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert st != 0 and b"current device" in lib.axb_last_error()
