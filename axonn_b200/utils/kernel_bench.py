"""Micro-benchmarks of the package's kernels against their roofline.

``python -m axonn_b200.utils.kernel_bench gemm`` times the tcgen05 GEMM on the
linear-layer shapes of the GPT-1.3B and Llama-8B configurations with CUDA
events (warm-up, L2 flushed between iterations) and prints achieved TFLOP/s
next to ``torch.matmul`` (cuBLAS) on the same operands.
"""

import json
import sys

import torch


def _flush_l2(buf):
    buf.zero_()


def time_cuda(fn, iters=10, warmup=3, flush=None):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        if flush is not None:
            _flush_l2(flush)
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        times.append(s.elapsed_time(e))
    times.sort()
    return times[len(times) // 2], times[0]


GEMM_SHAPES = [
    # (layout, M, N, K, label)
    ("nt", 16384, 6144, 2048, "gpt1.3b qkv fwd"),
    ("nt", 16384, 8192, 2048, "gpt1.3b fc1 fwd"),
    ("nt", 16384, 2048, 8192, "gpt1.3b fc2 fwd"),
    ("nn", 16384, 2048, 8192, "gpt1.3b fc1 dgrad"),
    ("tn", 8192, 2048, 16384, "gpt1.3b fc1 wgrad"),
    ("nt", 16384, 50304, 2048, "gpt1.3b lm head"),
    ("nt", 8192, 4096, 1024, "gpt1.3b fc1 r=c=2 local"),
    ("nt", 16384, 14336, 4096, "llama8b gate fwd"),
    ("nn", 16384, 4096, 14336, "llama8b gate dgrad"),
    ("tn", 14336, 4096, 16384, "llama8b gate wgrad"),
    ("nt", 8192, 8192, 8192, "square 8k"),
]


def bench_gemm(shapes=GEMM_SHAPES, iters=10):
    from axonn_b200 import ops

    dev = torch.device("cuda", 0)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    rows = []
    for layout, M, N, K, label in shapes:
        sa = (M, K) if layout != "tn" else (K, M)
        sb = (N, K) if layout == "nt" else (K, N)
        a = torch.randn(sa, device=dev, dtype=torch.bfloat16)
        b = torch.randn(sb, device=dev, dtype=torch.bfloat16)
        ours = {"nt": ops.matmul_nt, "nn": ops.matmul_nn, "tn": ops.matmul_tn}[layout]
        lib = {"nt": lambda: a @ b.t(), "nn": lambda: a @ b, "tn": lambda: a.t() @ b}[layout]
        out = torch.empty((M, N), device=dev, dtype=torch.bfloat16)
        t_ours, best_ours = time_cuda(lambda: ours(a, b, out=out), iters=iters, flush=flush)
        t_lib, best_lib = time_cuda(lib, iters=iters, flush=flush)
        fl = 2.0 * M * N * K
        rows.append(dict(label=label, layout=layout, M=M, N=N, K=K, ms=round(t_ours, 4),
                         tflops=round(fl / t_ours / 1e9, 1), best_tflops=round(fl / best_ours / 1e9, 1),
                         cublas_ms=round(t_lib, 4), cublas_tflops=round(fl / t_lib / 1e9, 1)))
        print(json.dumps(rows[-1]), flush=True)
        del a, b, out
    return rows


if __name__ == "__main__":
    what = sys.argv[1] if len(sys.argv) > 1 else "gemm"
    if what == "gemm":
        bench_gemm()
    else:
        raise SystemExit(f"unknown benchmark {what}")
