"""The output-arena allocator (csrc/arena.cu) is host-only code: first-fit with coalescing over a registered
address range.  Exercised here through its C symbols with a made-up base address (nothing is dereferenced)."""

import ctypes

import pytest

from axonn_b200.ops import _lib

MB = 1 << 20


def _lib_or_skip():
    if not _lib.available():
        pytest.skip("native library not built")
    L = _lib.lib()
    L.axb_arena_malloc.restype = ctypes.c_void_p
    L.axb_arena_malloc.argtypes = [ctypes.c_longlong, ctypes.c_int, ctypes.c_void_p]
    L.axb_arena_free.restype = None
    L.axb_arena_free.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_void_p]
    L.axb_arena_stat.restype = ctypes.c_ulonglong
    L.axb_arena_register.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_ulonglong]
    L.axb_arena_contains.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_ulonglong]
    return L


def test_arena_first_fit_coalesce_and_exhaustion():
    L = _lib_or_skip()
    dev, base, size = 63, 0x7000_0000_0000, 64 * MB     # device slot 63: never a real GPU in these tests
    assert L.axb_arena_register(dev, base, size) == 0
    a = L.axb_arena_malloc(10 * MB, dev, None)
    b = L.axb_arena_malloc(3 * MB, dev, None)            # rounded up to 4 MiB
    c = L.axb_arena_malloc(20 * MB, dev, None)
    assert a == base and b == base + 10 * MB and c == base + 14 * MB
    assert L.axb_arena_stat(dev, 0) == 34 * MB
    assert L.axb_arena_contains(dev, ctypes.c_void_p(c), 20 * MB) == 1
    assert L.axb_arena_contains(dev, ctypes.c_void_p(base + size - MB), 2 * MB) == 0
    assert L.axb_arena_malloc(40 * MB, dev, None) is None          # only 30 MiB left
    assert L.axb_arena_stat(dev, 3) == 1
    L.axb_arena_free(a, 0, dev, None)
    L.axb_arena_free(b, 0, dev, None)                    # a and b coalesce into one 14 MiB hole
    d = L.axb_arena_malloc(14 * MB, dev, None)
    assert d == base
    L.axb_arena_free(c, 0, dev, None)
    L.axb_arena_free(d, 0, dev, None)
    assert L.axb_arena_stat(dev, 0) == 0 and L.axb_arena_stat(dev, 4) == 64 * MB
    assert L.axb_arena_stat(dev, 1) == 34 * MB           # high-water mark
    L.axb_arena_free(ctypes.c_void_p(base + 2 * MB), 0, dev, None)  # unknown pointer: ignored
    assert L.axb_arena_stat(dev, 0) == 0
    assert L.axb_arena_register(dev, None, 0) == 0
