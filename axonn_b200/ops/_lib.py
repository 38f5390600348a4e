"""Loader for the in-tree CUDA library (``axonn_b200/lib/libaxonn_b200.so``).

The kernels are plain ``extern "C"`` launchers compiled by nvcc for sm_100a
(see ``axonn_b200/utils/build.py``); they are called through ctypes with raw
device pointers and the current CUDA stream, so the library has no dependency
on the PyTorch C++ ABI.  On a machine with a GPU a missing library is an error,
never a silent fallback.
"""

import ctypes
import os
import threading

import torch

_LIB = None
_LOCK = threading.Lock()
LIB_DIR = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "lib")
LIB_PATH = os.path.join(LIB_DIR, "libaxonn_b200.so")

# number of kernels launched through this library since the last reset
launch_count = 0


class KernelError(RuntimeError):
    pass


def available() -> bool:
    return os.path.exists(LIB_PATH)


def lib():
    """Return the loaded library, building it first when it is missing and nvcc
    is present."""
    global _LIB
    if _LIB is not None:
        return _LIB
    with _LOCK:
        if _LIB is None:
            if not os.path.exists(LIB_PATH):
                from ..utils import build

                build.build_library(verbose=False)
            _LIB = ctypes.CDLL(LIB_PATH, mode=ctypes.RTLD_GLOBAL)
            _LIB.axb_last_error.restype = ctypes.c_char_p
    return _LIB


def use_cuda_kernels(*tensors) -> bool:
    """True when the operands live on a GPU (then the library is mandatory)."""
    return len(tensors) > 0 and all(t is None or t.is_cuda for t in tensors) and any(
        t is not None for t in tensors)


def stream_ptr() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def ptr(t) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def check(status: int, what: str):
    global launch_count
    if status != 0:
        msg = lib().axb_last_error()
        raise KernelError(f"{what} failed (status {status}): {msg.decode() if msg else ''}")
    launch_count += 1


def add_launches(n: int):
    global launch_count
    launch_count += n


def reset_launch_count():
    global launch_count
    launch_count = 0
