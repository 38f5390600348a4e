"""Matrix products of the tensor-parallel layers.

Three layouts cover forward, input-gradient and weight-gradient of a linear
layer without any transposed copies:

    matmul_nt(a[M,K], b[N,K]) = a @ b.T      forward      (K-major x K-major)
    matmul_nn(a[M,K], b[K,N]) = a @ b        input grad   (K-major x N-major)
    matmul_tn(a[K,M], b[K,N]) = a.T @ b      weight grad  (M-major x N-major)

On CUDA (bf16/fp16 operands) these run on the package's tcgen05 kernel
(``csrc/gemm_tcgen05.cu``: TMA-fed shared-memory pipeline, ``tcgen05.mma`` into
TMEM accumulators, warp-specialised persistent CTAs) with optional fused
epilogues (bias add, GELU, fp32 output, ``+=`` accumulate).  On CPU they are
``torch.matmul``.  They replace ``input_.matmul(weight.t())``,
``grad_output.matmul(weight)`` and ``grad_output.t().mm(input_)`` of the
reference's ``axonn/intra_layer/fully_connected.py:118,140,147-151``.
"""

import ctypes

import torch

from . import _lib

EPI_NONE, EPI_BIAS, EPI_BIAS_GELU, EPI_GELU = 0, 1, 2, 3
_DT = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}


def _cuda_ok(a, b):
    """Kernel path: 16-bit CUDA operands whose dimensions give 16-byte aligned TMA
    row pitches.  Odd shapes (e.g. a router with 4 outputs) use torch.matmul."""
    if not (a.is_cuda and b.is_cuda and a.dtype == b.dtype and a.dtype in (torch.bfloat16, torch.float16)):
        return False
    # every dimension that is a contiguous (innermost) extent or the output width
    return a.shape[1] % 8 == 0 and b.shape[1] % 8 == 0 and b.shape[0] % 8 == 0


def _rowmajor(t):
    """Contiguous 2-D view (copy only when strides are not already dense)."""
    return t if t.is_contiguous() else t.contiguous()


def _launch(layout, a, b, M, N, K, out, bias=None, epilogue=EPI_NONE, accumulate=False, aux=None):
    if K % 8 or N % 8 or (layout == 2 and M % 8):
        raise ValueError(f"gemm dims must be multiples of 8 for 16-byte TMA strides, got M={M} N={N} K={K}")
    L = _lib.lib()
    st = L.axb_gemm(
        ctypes.c_int(layout), _lib.ptr(a), _lib.ptr(b), _lib.ptr(out), _lib.ptr(bias), _lib.ptr(aux),
        ctypes.c_int(M), ctypes.c_int(N), ctypes.c_int(K),
        ctypes.c_int(_DT[a.dtype]), ctypes.c_int(_DT[out.dtype]),
        ctypes.c_int(epilogue), ctypes.c_int(1 if accumulate else 0),
        ctypes.c_int(a.device.index), _lib.stream_ptr())
    _lib.check(st, "axb_gemm")
    return out


def matmul_nt(a, b, bias=None, epilogue=EPI_NONE, out_dtype=None, out=None, accumulate=False, aux=None):
    """``a[M,K] @ b[N,K].T`` (+bias, +GELU).  ``aux`` (same shape as the output)
    receives the pre-activation when the epilogue applies GELU."""
    M, K = a.shape
    N = b.shape[0]
    assert b.shape[1] == K
    if _cuda_ok(a, b):
        a, b = _rowmajor(a), _rowmajor(b)
        if out is None:
            out = torch.empty((M, N), dtype=out_dtype or a.dtype, device=a.device)
        return _launch(0, a, b, M, N, K, out, bias, epilogue, accumulate, aux)
    if a.is_cuda and a.dtype != b.dtype:
        raise TypeError("matmul_nt: operand dtypes differ")
    y = torch.matmul(a, b.t())
    if epilogue in (EPI_BIAS, EPI_BIAS_GELU):
        y = y + bias
    if epilogue in (EPI_BIAS_GELU, EPI_GELU):
        if aux is not None:
            aux.copy_(y)
        y = torch.nn.functional.gelu(y, approximate="tanh")
    if out_dtype is not None:
        y = y.to(out_dtype)
    if out is not None:
        if accumulate:
            out.add_(y)
        else:
            out.copy_(y)
        return out
    return y


def matmul_nn(a, b, out_dtype=None, out=None, accumulate=False):
    """``a[M,K] @ b[K,N]``."""
    M, K = a.shape
    N = b.shape[1]
    assert b.shape[0] == K
    if _cuda_ok(a, b):
        a, b = _rowmajor(a), _rowmajor(b)
        if out is None:
            out = torch.empty((M, N), dtype=out_dtype or a.dtype, device=a.device)
        return _launch(1, a, b, M, N, K, out, accumulate=accumulate)
    y = torch.matmul(a, b)
    if out_dtype is not None:
        y = y.to(out_dtype)
    if out is not None:
        return out.add_(y) if accumulate else out.copy_(y)
    return y


def matmul_tn(a, b, out_dtype=None, out=None, accumulate=False):
    """``a[K,M].T @ b[K,N]`` (reduction over the leading dimension of both)."""
    K, M = a.shape
    N = b.shape[1]
    assert b.shape[0] == K
    if _cuda_ok(a, b):
        a, b = _rowmajor(a), _rowmajor(b)
        if out is None:
            out = torch.empty((M, N), dtype=out_dtype or a.dtype, device=a.device)
        return _launch(2, a, b, M, N, K, out, accumulate=accumulate)
    y = torch.matmul(a.t(), b)
    if out_dtype is not None:
        y = y.to(out_dtype)
    if out is not None:
        return out.add_(y) if accumulate else out.copy_(y)
    return y


def _batched_ok(a, b):
    return (a.is_cuda and b.is_cuda and a.dtype == b.dtype and a.dtype in (torch.bfloat16, torch.float16)
            and a.shape[-1] % 8 == 0 and b.shape[-1] % 8 == 0 and b.shape[-2] % 8 == 0
            and hasattr(_lib.lib(), "axb_gemm_batched"))


def _launch_batched(layout, a, b, nb, M, N, K, out, seg=None, seg_rows=0):
    L = _lib.lib()
    nseg = 0
    if seg is not None:
        assert seg.dtype == torch.int32 and seg.is_cuda and seg.is_contiguous() and seg.shape[0] == nb
        nseg = seg.shape[1]
    st = L.axb_gemm_batched(
        ctypes.c_int(layout), _lib.ptr(a), _lib.ptr(b), _lib.ptr(out), ctypes.c_int(nb), ctypes.c_int(M),
        ctypes.c_int(N), ctypes.c_int(K), ctypes.c_int(a.shape[1]), ctypes.c_int(b.shape[1]), ctypes.c_int(M),
        ctypes.c_int(_DT[a.dtype]), ctypes.c_int(_DT[out.dtype]), ctypes.c_int(0),
        _lib.ptr(seg), ctypes.c_int(seg_rows), ctypes.c_int(nseg),
        ctypes.c_int(a.device.index), _lib.stream_ptr())
    _lib.check(st, "axb_gemm_batched")
    return out


def bmm_nt(a, b, out_dtype=None, seg=None, seg_rows=0):
    """``a[E,M,K] @ b[E,N,K].T`` per problem ``E``: one launch of the CTA-pair kernel over all problems' tiles.
    ``seg`` / ``seg_rows``: row mask over M (see ``ops.linear_batched``)."""
    E, M, K = a.shape
    N = b.shape[1]
    if _batched_ok(a, b):
        a, b = _rowmajor(a), _rowmajor(b)
        out = torch.empty((E, M, N), dtype=out_dtype or a.dtype, device=a.device)
        return _launch_batched(0, a, b, E, M, N, K, out, seg, seg_rows)
    y = torch.matmul(a, b.transpose(1, 2))
    return y if out_dtype is None else y.to(out_dtype)


def bmm_nn(a, b, out_dtype=None, seg=None, seg_rows=0):
    """``a[E,M,K] @ b[E,K,N]`` per problem; row mask over M."""
    E, M, K = a.shape
    N = b.shape[2]
    if _batched_ok(a, b) and K % 64 == 0:
        a, b = _rowmajor(a), _rowmajor(b)
        out = torch.empty((E, M, N), dtype=out_dtype or a.dtype, device=a.device)
        return _launch_batched(1, a, b, E, M, N, K, out, seg, seg_rows)
    y = torch.matmul(a, b)
    return y if out_dtype is None else y.to(out_dtype)


def bmm_tn(a, b, out_dtype=None, seg=None, seg_rows=0):
    """``a[E,K,M].T @ b[E,K,N]`` per problem (reduction over the rows of both); row mask over K."""
    E, K, M = a.shape
    N = b.shape[2]
    if _batched_ok(a, b) and K % 64 == 0:
        a, b = _rowmajor(a), _rowmajor(b)
        out = torch.empty((E, M, N), dtype=out_dtype or a.dtype, device=a.device)
        return _launch_batched(2, a, b, E, M, N, K, out, seg, seg_rows)
    y = torch.matmul(a.transpose(1, 2), b)
    return y if out_dtype is None else y.to(out_dtype)
