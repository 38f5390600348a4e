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


def bench_attention(small=False):
    """tcgen05 flash-attention forward vs cuDNN SDPA forward on packed QKV."""
    import math

    import torch.nn.functional as F

    from axonn_b200.ops.attention_cuda import flash_fwd_packed

    dev = torch.device("cuda", 0)
    cases = [(4, 2048, 8, 1, 128)] if small else [(8, 2048, 16, 1, 128), (4, 4096, 8, 4, 128), (8, 2048, 16, 1, 64)]
    for B, S, G, qpk, D in cases:
        qkv = torch.randn(B, S, G, qpk + 2, D, device=dev, dtype=torch.bfloat16)
        scale = 1.0 / math.sqrt(D)
        q = qkv[:, :, :, :qpk].reshape(B, S, G * qpk, D).transpose(1, 2).contiguous()
        k = qkv[:, :, :, qpk].transpose(1, 2).repeat_interleave(qpk, dim=1).contiguous()
        v = qkv[:, :, :, qpk + 1].transpose(1, 2).repeat_interleave(qpk, dim=1).contiguous()
        t_ours, _ = time_cuda(lambda: flash_fwd_packed(qkv, scale), iters=3 if small else 10)
        t_lib, _ = time_cuda(lambda: F.scaled_dot_product_attention(q, k, v, is_causal=True), iters=3 if small else 10)
        fl = 4.0 * B * G * qpk * S * S * D / 2
        from axonn_b200.ops.attention_cuda import flash_bwd_packed

        out, lse = flash_fwd_packed(qkv, scale)
        d_out = torch.randn_like(out)
        t_bwd, _ = time_cuda(lambda: flash_bwd_packed(qkv, out, d_out, lse, scale), iters=3 if small else 10)
        qr, kr, vr = (t.detach().requires_grad_(True) for t in (q, k, v))
        o_ref = F.scaled_dot_product_attention(qr, kr, vr, is_causal=True)
        g_ref = torch.randn_like(o_ref)
        t_lib_bwd, _ = time_cuda(lambda: torch.autograd.grad(o_ref, (qr, kr, vr), g_ref, retain_graph=True),
                                 iters=3 if small else 10)
        import os

        if int(os.environ.get("AXB_FA_DEBUG", "0")) & 4:
            from axonn_b200.ops import _lib

            w = {i: _lib.lib().axb_debug_word(0, i, 1) for i in (2, 3, 4, 7, 8, 9, 10, 11, 12, 13)}
            n = max(1, w[7])
            print("bwd CTA (0,0,0), us per iteration: MMA warp waits: Q/dO %.2f, S columns free %.2f, P/dS %.2f | "
                  "softmax warp: wait S/dP %.2f, P/dS math %.2f, wait dQ %.2f, dQ reduction %.2f (TMEM -> smem done at %.2f, "
                  "bulk reduce issued at %.2f) (%d iterations)" % (
                      w[2] / n / 1e3, w[3] / n / 1e3, w[4] / n / 1e3, w[8] / n / 1e3, w[9] / n / 1e3,
                      w[10] / n / 1e3, w[11] / n / 1e3, w[12] / n / 1e3, w[13] / n / 1e3, n), flush=True)
        print(json.dumps(dict(B=B, S=S, heads=G * qpk, kv_heads=G, D=D, ms=round(t_ours, 4),
                              tflops=round(fl / t_ours / 1e9, 1), cudnn_ms=round(t_lib, 4),
                              cudnn_tflops=round(fl / t_lib / 1e9, 1), bwd_ms=round(t_bwd, 4),
                              bwd_tflops=round(2.5 * fl / t_bwd / 1e9, 1), cudnn_bwd_ms=round(t_lib_bwd, 4))),
              flush=True)


FUSED_SHAPES = [
    # (M, N, K, label) per-rank GEMM of the GPT-1.3B r=c=d=2 configuration, one 32-sequence microbatch
    (65536, 4096, 1024, "fc1 fwd + AR(c)"),
    (65536, 3072, 1024, "qkv fwd + AR(c)"),
    (65536, 1024, 4096, "fc2 fwd + AR(r)"),
    (65536, 1024, 1024, "proj fwd + AR(r)"),
    (16384, 4096, 1024, "fc1 fwd + AR, 8 sequences"),
]


def bench_fused(iters=8):
    """Fused GEMM+all-reduce vs GEMM followed by an NCCL all-reduce, on the ranks of the default group.
    Roofline: max(FLOPs / measured bf16 peak, bytes over NVLink / 770 GB/s), bytes = M*N*2 per direction."""
    import torch.distributed as dist

    from axonn_b200 import ops
    from axonn_b200.metrics import measured_peaks
    from axonn_b200.parallel import fused

    rank, world = dist.get_rank(), dist.get_world_size()
    dev = torch.device("cuda", torch.cuda.current_device())
    peak, _, kind = measured_peaks()
    group = dist.group.WORLD
    import os

    shapes = FUSED_SHAPES[:1] if os.environ.get("AXB_AR_DEBUG") else FUSED_SHAPES
    for M, N, K, label in shapes:
        a = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
        b = torch.randn(N, K, device=dev, dtype=torch.bfloat16)

        def run_fused():
            return fused.gemm_all_reduce(0, a, b, group)

        def run_unfused():
            out = ops.matmul_nt(a, b)
            dist.all_reduce(out, group=group)
            return out

        def run_gemm_only():
            return ops.matmul_nt(a, b)

        res = {}
        for name, fn in (("fused", run_fused), ("gemm+nccl", run_unfused), ("gemm", run_gemm_only)):
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            dist.barrier()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            for _ in range(iters):
                fn()
            e.record()
            torch.cuda.synchronize()
            t = torch.tensor([s.elapsed_time(e) / iters], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            res[name] = float(t.item())
        flops, nbytes = 2.0 * M * N * K, 2.0 * M * N * (world - 1)
        roof_ms = max(flops / (peak * 1e12), nbytes / 770e9) * 1e3
        if rank == 0:
            print(json.dumps(dict(label=label, M=M, N=N, K=K, ranks=world, fused_ms=round(res["fused"], 4),
                                  gemm_nccl_ms=round(res["gemm+nccl"], 4), gemm_ms=round(res["gemm"], 4),
                                  roofline_ms=round(roof_ms, 4), fraction=round(roof_ms / res["fused"], 3),
                                  nvlink_gbs=round(nbytes / res["fused"] / 1e6, 1), peak=f"{peak} TFLOP/s {kind}")),
                  flush=True)
        del a, b


def bench_memory_bound(rows=16384, H=2048):
    """Memory-bound kernels against the measured copy bandwidth: algorithmic bytes / CUDA-event time."""
    from axonn_b200 import ops
    from axonn_b200.metrics import measured_peaks

    dev = torch.device("cuda", 0)
    _, hbm, kind = measured_peaks()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    x = torch.randn(rows, H, device=dev).bfloat16().requires_grad_(True)
    g = torch.ones(H, device=dev).bfloat16().requires_grad_(True)
    b = torch.zeros(H, device=dev).bfloat16().requires_grad_(True)
    dy = torch.randn(rows, H, device=dev).bfloat16()
    out = []

    def report(label, ms, nbytes):
        gbs = nbytes / ms / 1e6
        out.append(dict(label=label, rows=rows, H=H, ms=round(ms, 4), gbs=round(gbs, 1),
                        fraction=round(gbs / hbm, 3), peak=f"{hbm} GB/s {kind}"))
        print(json.dumps(out[-1]), flush=True)

    nb = rows * H * 2
    for name, fn in (("layernorm", lambda: ops.layer_norm(x, g, b, 1e-5)), ("rmsnorm", lambda: ops.rms_norm(x, g, 1e-5))):
        with torch.no_grad():
            t, _ = time_cuda(fn, flush=flush)
        report(name + " fwd", t, 2 * nb)
        y = fn()
        t, _ = time_cuda(lambda: torch.autograd.grad(y, (x, g), dy, retain_graph=True), flush=flush)
        report(name + " bwd (dx, dgamma, dbeta)", t, 3 * nb)
    with torch.no_grad():
        t, _ = time_cuda(lambda: ops.column_sum(dy), flush=flush)
        report("column sum (bias gradient)", t, nb)
        t, _ = time_cuda(lambda: dy.sum(0, dtype=torch.float32), flush=flush)
        report("column sum, torch reduce", t, nb)
    h = torch.randn(rows, 4 * H, device=dev).bfloat16().requires_grad_(True)
    dh = torch.randn_like(h)
    with torch.no_grad():
        t, _ = time_cuda(lambda: ops.gelu(h), flush=flush)
    report("gelu fwd", t, 2 * 4 * nb)
    yh = ops.gelu(h)
    t, _ = time_cuda(lambda: torch.autograd.grad(yh, h, dh, retain_graph=True), flush=flush)
    report("gelu bwd", t, 3 * 4 * nb)
    with torch.no_grad():
        t, _ = time_cuda(lambda: ops.gelu_backward_colsum(dh, h.detach()), flush=flush)
    report("gelu bwd + column sums (bias gradient)", t, 3 * 4 * nb)
    return out


def bench_fused_loopback(M=16384, N=4096, K=1024, iters=3):
    """One-GPU emulation of the two-rank fused GEMM+all-reduce (peer slots aliased onto local memory): the
    local cost of the communication path - epilogue pushes, flags, reducer warps - without NVLink."""
    from axonn_b200 import ops
    from axonn_b200.parallel import fused

    dev = torch.device("cuda", 0)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    a = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
    b = torch.randn(N, K, device=dev, dtype=torch.bfloat16)
    t_loop, _ = time_cuda(lambda: fused.gemm_all_reduce_loopback(a, b), iters=iters, flush=flush)
    t_gemm, _ = time_cuda(lambda: ops.matmul_nt(a, b), iters=iters, flush=flush)
    ref = 2.0 * (a.float() @ b.float().t())
    err = float((fused.gemm_all_reduce_loopback(a, b).float() - ref).abs().max() / ref.abs().max())
    import os

    if int(os.environ.get("AXB_AR_DEBUG", "0")) & 64:
        from axonn_b200.ops import _lib

        w = {i: _lib.lib().axb_debug_word(0, i, 1) for i in (2, 3, 7)}
        print("reducer of CTA 0, last call: wait %.2f us/tile, work %.2f us/tile, %d tiles" % (
            w[2] / max(1, w[7]) / 1e3, w[3] / max(1, w[7]) / 1e3, w[7]), flush=True)
    print(json.dumps(dict(label="fused GEMM+AR, two ranks emulated on one GPU", M=M, N=N, K=K,
                          loopback_ms=round(t_loop, 4), gemm_ms=round(t_gemm, 4), rel_err=round(err, 5))), flush=True)


if __name__ == "__main__":
    what = sys.argv[1] if len(sys.argv) > 1 else "gemm"
    if what == "gemm":
        bench_gemm()
    elif what == "gemm_small":
        # one mid-size shape (working set 192 MB > L2), a handful of launches: the case profiled with ncu
        bench_gemm(shapes=[("nt", 8192, 8192, 2048, "profile case")], iters=3)
    elif what == "attn_small":
        bench_attention(small=True)
    elif what == "attn":
        bench_attention()
    elif what == "memory":
        bench_memory_bound()
    elif what == "fused_loopback":
        bench_fused_loopback()
    elif what == "fused":
        import os

        import torch.distributed as dist

        local = int(os.environ.get("LOCAL_RANK", 0))
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        bench_fused()
        dist.destroy_process_group()
    else:
        raise SystemExit(f"unknown benchmark {what}")
