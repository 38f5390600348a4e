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
# AXONN_LIB_PATH selects a library built elsewhere (e.g. an ablation build with -DAXB_ABLATION);
# AXONN_DEBUG_BOUNDS=1 selects the bounds-checking build when it has been built
# (``python axonn_b200/utils/build.py --debug-bounds``)
_DEBUG_LIB = os.path.join(LIB_DIR, "libaxonn_b200_debug.so")
LIB_PATH = os.environ.get("AXONN_LIB_PATH") or (
    _DEBUG_LIB if os.environ.get("AXONN_DEBUG_BOUNDS", "0") not in ("", "0") and os.path.exists(_DEBUG_LIB)
    else os.path.join(LIB_DIR, "libaxonn_b200.so"))

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
            ms = os.environ.get("AXONN_COMM_TIMEOUT_MS")
            if ms:
                _LIB.axb_set_wait_timeout_ms(ctypes.c_uint(int(ms)))
    return _LIB


def set_wait_timeout_ms(ms: int):
    """Deadline of every device-side wait (mbarrier, peer flag).  A kernel whose wait runs out returns and
    reports through the status word (``check_status``).  Default 120000 ms; ``AXONN_COMM_TIMEOUT_MS`` sets it
    at load time."""
    lib().axb_set_wait_timeout_ms(ctypes.c_uint(int(ms)))


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


_STATUS_NAMES = {
    0x101: "GEMM producer: shared-memory stage never freed",
    0x102: "GEMM MMA issuer: operand stage or accumulator never arrived",
    0x104: "GEMM epilogue: accumulator never completed",
    0x108: "fused GEMM: a peer never finished the previous call on this buffer",
    0x110: "all-gather stage: a peer never published its weight shard",
    0x120: "fused reduction: aborted while waiting for partial tiles",
    0x121: "fused reduction: partial tiles of a peer never arrived",
    0x122: "fused reduction (shared-memory ring): inbox slots never arrived",
    0x123: "fused reduction (shared-memory ring): ring group never freed",
    0x109: "fused all-reduce (two-shot): a peer never finished writing its rows of the result",
    0x124: "fused all-reduce (two-shot): a peer never announced where its output lies",
    0x201: "expert dispatch / combine: a peer never signalled",
    0x301: "gradient all-reduce: a peer never published its bucket",
    0x302: "gradient all-reduce: a peer never delivered its partial slices",
    0x303: "gradient all-reduce: a peer never delivered its reduced slice",
    0x501: "row all-to-all: a peer never announced its output",
    0x502: "row all-to-all / embedding rows: a peer never finished",
    0x503: "embedding row fetch: a peer never published its table shard",
    0x504: "embedding gradient: a peer never published its gradient shard",
    0x701: "bounds check (debug build): inbox slot outside the peer's inbox",
    0x702: "bounds check (debug build): output element outside C",
    0x703: "bounds check (debug build): flag index outside the flag array",
    0x401: "flash attention forward: producer timed out",
    0x402: "flash attention forward: MMA issuer timed out",
    0x404: "flash attention forward: softmax warps timed out",
    0x411: "flash attention backward: producer timed out",
    0x412: "flash attention backward: MMA issuer timed out",
    0x414: "flash attention backward: softmax / reduction warps timed out",
    0x141: "CTA-pair GEMM producer timed out",
    0x142: "CTA-pair GEMM MMA issuer timed out",
    0x144: "CTA-pair GEMM epilogue timed out",
}


class AxonnCommTimeout(KernelError):
    """A device-side wait (mbarrier or peer flag) ran into its deadline; ``status`` is the kernel's reason code."""

    def __init__(self, status: int):
        self.status = status
        super().__init__(f"device-side wait timed out (status 0x{status:x}: {_STATUS_NAMES.get(status, 'unknown')})")


def device_status(device=None, clear=True) -> int:
    """Status word that kernels write when one of their bounded waits gave up (0: none did).  The word lives
    in mapped host memory, so reading it needs no synchronisation; it is meaningful once the kernels in
    question have finished (e.g. after reading the loss)."""
    import torch

    if not available() or not torch.cuda.is_available():
        return 0
    dev = torch.cuda.current_device() if device is None else int(device)
    return int(lib().axb_device_status(ctypes.c_int(dev), ctypes.c_int(1 if clear else 0)))


def check_status(device=None):
    """Raise ``AxonnCommTimeout`` (a ``KernelError``) if a kernel on ``device`` reported a timed-out wait since
    the last check."""
    st = device_status(device, clear=True)
    if st not in (0, 0xFFFFFFFF):
        raise AxonnCommTimeout(st)
