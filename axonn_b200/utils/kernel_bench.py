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


def _timed_group(fn, iters, dev):
    """ms per call: CUDA events around ``iters`` back-to-back calls after 3 warm-up calls, max over ranks."""
    import torch.distributed as dist

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
    return float(t.item())


def bench_fused(iters=8, two_shot=True):
    """Fused GEMM+all-reduce vs GEMM followed by an NCCL all-reduce, on the ranks of the default group.
    ``two_shot``: outputs in the peer-mapped arena, every 32-row unit reduced by one owner (the default of the
    layers); otherwise the one-shot form.  Roofline: max(FLOPs / measured bf16 peak, bytes leaving a rank over
    NVLink / 770 GB/s); bytes = M*N*2 * (n-1) one-shot, M*N*2 * 2(n-1)/n two-shot."""
    import torch.distributed as dist

    from axonn_b200 import ops
    from axonn_b200.metrics import measured_peaks
    from axonn_b200.parallel import fused, symm

    rank, world = dist.get_rank(), dist.get_world_size()
    dev = torch.device("cuda", torch.cuda.current_device())
    peak, _, kind = measured_peaks()
    group = dist.group.WORLD
    if two_shot:
        assert symm.create_output_arena(4 << 30) is not None, "no output arena"
    for M, N, K, label in FUSED_SHAPES:
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
            res[name] = _timed_group(fn, iters, dev)
        flops = 2.0 * M * N * K
        nbytes = 2.0 * M * N * (2.0 * (world - 1) / world if two_shot else (world - 1))
        roof_ms = max(flops / (peak * 1e12), nbytes / 770e9) * 1e3
        if rank == 0:
            print(json.dumps(dict(label=label, protocol="two-shot" if two_shot else "one-shot", M=M, N=N, K=K,
                                  ranks=world, fused_ms=round(res["fused"], 4),
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
    t_two, _ = time_cuda(lambda: fused.gemm_all_reduce_loopback(a, b, two_shot=True), iters=iters, flush=flush)
    print(json.dumps(dict(label="fused GEMM+AR, two ranks emulated on one GPU", M=M, N=N, K=K,
                          loopback_ms=round(t_loop, 4), two_shot_loopback_ms=round(t_two, 4),
                          gemm_ms=round(t_gemm, 4), rel_err=round(err, 5))), flush=True)


def bench_fused_loopback_two_shot(M=16384, N=4096, K=1024, iters=3):
    """Only the two-shot kernel of the one-GPU emulation (3 warm-up + 3 timed launches of one kernel): the
    case that is captured with ncu (``-k regex:gemm_tcgen05 -s 3 -c 1``)."""
    from axonn_b200.parallel import fused

    dev = torch.device("cuda", 0)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    a = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
    b = torch.randn(N, K, device=dev, dtype=torch.bfloat16)
    t_two, _ = time_cuda(lambda: fused.gemm_all_reduce_loopback(a, b, two_shot=True), iters=iters, flush=flush)
    print(json.dumps(dict(label="fused GEMM+AR two-shot, rank 0 of 2 emulated on one GPU", M=M, N=N, K=K,
                          two_shot_loopback_ms=round(t_two, 4))), flush=True)


AG_SHAPES = [
    # (tokens, out_l, in_l, label): weight [out_l, in_l] sharded by rows over the ranks of the group
    (16384, 28672, 4096, "Llama-8B gate|up fwd"),
    (16384, 4096, 14336, "Llama-8B down fwd"),
    (16384, 6144, 4096, "Llama-8B qkv fwd"),
    (16384, 8192, 2048, "GPT-1.3B fc1 fwd"),
]


def bench_ag(iters=6):
    """Fused all-gather -> GEMM (weight shards pulled over NVLink inside the GEMM kernel) against an NCCL
    all-gather followed by the plain GEMM, and the plain GEMM alone, on the ranks of the default group.
    Forward (A W^T) and input-gradient (A W) products.  Roofline: max(FLOPs / measured bf16 peak, bytes a rank
    pulls over NVLink / 770 GB/s)."""
    import torch.distributed as dist

    from axonn_b200 import ops
    from axonn_b200.metrics import measured_peaks
    from axonn_b200.parallel import fused

    rank, world = dist.get_rank(), dist.get_world_size()
    dev = torch.device("cuda", torch.cuda.current_device())
    peak, _, kind = measured_peaks()
    group = dist.group.WORLD
    for T, out_l, in_l, label in AG_SHAPES:
        if (out_l // world) % 128 or out_l % world:
            continue
        shard = (torch.randn(out_l // world, in_l, device=dev) * 0.05).bfloat16().reshape(-1)
        full = torch.empty(out_l * in_l, device=dev, dtype=torch.bfloat16)
        for layout, tag in ((0, "fwd  x W^T"), (1, "dgrad g W")):
            a = torch.randn(T, in_l if layout == 0 else out_l, device=dev, dtype=torch.bfloat16)

            def run_fused():
                return fused.all_gather_gemm(layout, a, shard, group, (out_l, in_l))[0]

            def run_unfused():
                dist.all_gather_into_tensor(full, shard, group=group)
                w = full.view(out_l, in_l)
                return ops.matmul_nt(a, w) if layout == 0 else ops.matmul_nn(a, w)

            def run_gemm_only():
                w = full.view(out_l, in_l)
                return ops.matmul_nt(a, w) if layout == 0 else ops.matmul_nn(a, w)

            res = {n_: _timed_group(f, iters, dev) for n_, f in (("fused", run_fused), ("nccl+gemm", run_unfused),
                                                                  ("gemm", run_gemm_only))}
            flops = 2.0 * T * out_l * in_l
            nbytes = 2.0 * out_l * in_l * (world - 1) / world
            roof_ms = max(flops / (peak * 1e12), nbytes / 770e9) * 1e3
            if rank == 0:
                print(json.dumps(dict(label=f"{label} ({tag})", tokens=T, out_l=out_l, in_l=in_l, ranks=world,
                                      fused_ms=round(res["fused"], 4), nccl_gemm_ms=round(res["nccl+gemm"], 4),
                                      gemm_ms=round(res["gemm"], 4), roofline_ms=round(roof_ms, 4),
                                      fraction=round(roof_ms / res["fused"], 3), peak=f"{peak} TFLOP/s {kind}")),
                      flush=True)
            del a
        del shard, full


def bench_rs(iters=6):
    """Fused weight-gradient GEMM -> reduce-scatter against GEMM + NCCL reduce_scatter_tensor."""
    import torch.distributed as dist

    from axonn_b200 import ops
    from axonn_b200.metrics import measured_peaks
    from axonn_b200.parallel import fused

    rank, world = dist.get_rank(), dist.get_world_size()
    dev = torch.device("cuda", torch.cuda.current_device())
    peak, _, kind = measured_peaks()
    group = dist.group.WORLD
    for T, out_l, in_l, label in [(16384, 14336, 4096, "Llama-8B gate wgrad"), (16384, 4096, 4096, "Llama-8B o wgrad"),
                                  (16384, 8192, 2048, "GPT-1.3B fc1 wgrad")]:
        if out_l % world or (out_l // world) % 32:
            continue
        dy = torch.randn(T, out_l, device=dev, dtype=torch.bfloat16)
        x = torch.randn(T, in_l, device=dev, dtype=torch.bfloat16)
        shard = torch.empty(out_l // world, in_l, device=dev, dtype=torch.bfloat16)

        def run_fused():
            return fused.gemm_reduce_scatter(2, dy, x, group)

        def run_unfused():
            gw = ops.matmul_tn(dy, x)
            dist.reduce_scatter_tensor(shard, gw, group=group)
            return shard

        def run_gemm_only():
            return ops.matmul_tn(dy, x)

        res = {n_: _timed_group(f, iters, dev) for n_, f in (("fused", run_fused), ("gemm+nccl", run_unfused),
                                                              ("gemm", run_gemm_only))}
        flops = 2.0 * T * out_l * in_l
        nbytes = 2.0 * out_l * in_l * (world - 1) / world
        roof_ms = max(flops / (peak * 1e12), nbytes / 770e9) * 1e3
        if rank == 0:
            print(json.dumps(dict(label=label, tokens=T, out_l=out_l, in_l=in_l, ranks=world,
                                  fused_ms=round(res["fused"], 4), gemm_nccl_ms=round(res["gemm+nccl"], 4),
                                  gemm_ms=round(res["gemm"], 4), roofline_ms=round(roof_ms, 4),
                                  fraction=round(roof_ms / res["fused"], 3), peak=f"{peak} TFLOP/s {kind}")),
                  flush=True)
        del dy, x, shard


def bench_grad_ar(iters=6):
    """Peer-memory gradient all-reduce (+scale) of a list of tensors against flatten + NCCL all-reduce + scale +
    unflatten.  Roofline: 2 (n-1)/n of the bytes over NVLink at 770 GB/s per direction."""
    import torch.distributed as dist

    from axonn_b200 import ops

    rank, world = dist.get_rank(), dist.get_world_size()
    dev = torch.device("cuda", torch.cuda.current_device())
    group = dist.group.WORLD
    for dtype in (torch.bfloat16, torch.float32):
        grads = [torch.randn(n, device=dev).to(dtype) for n in [4096 * 4096] * 24 + [4096] * 48 + [50304 * 512]]
        nbytes = sum(g.numel() * g.element_size() for g in grads)

        def run_ours():
            ops.all_reduce_bucketed_(grads, group, scale=1.0 / world)

        def run_nccl():
            flat = torch._utils._flatten_dense_tensors(grads)
            dist.all_reduce(flat, group=group)
            flat.mul_(1.0 / world)
            for old, new in zip(grads, torch._utils._unflatten_dense_tensors(flat, grads)):
                old.copy_(new)

        res = {n_: _timed_group(f, iters, dev) for n_, f in (("ours", run_ours), ("nccl", run_nccl))}
        roof_ms = 2.0 * (world - 1) / world * nbytes / 770e9 * 1e3
        if rank == 0:
            print(json.dumps(dict(label="gradient all-reduce + scale", dtype=str(dtype), mbytes=round(nbytes / 2**20, 1),
                                  tensors=len(grads), ranks=world, ours_ms=round(res["ours"], 4),
                                  nccl_flat_ms=round(res["nccl"], 4), roofline_ms=round(roof_ms, 4),
                                  fraction=round(roof_ms / res["ours"], 3))), flush=True)
        del grads


def bench_moe(iters=5, tokens=8192, hidden=4096, ffn=14336, n_experts=8, top_k=2):
    """Expert-parallel MoE layer (Mixtral-8x7B layer shape: 8192 tokens per GPU, top-2 of 8 experts), forward +
    backward, on the ranks of the default group: peer-memory dispatch / combine kernels against NCCL
    ``all_to_all_single``, and the expert GEMMs as one batched launch per GEMM against one launch per expert."""
    import torch.distributed as dist

    from .. import axonn as ax
    from .. import ops
    from ..parallel import moe, moe_kernels

    world, rank = dist.get_world_size(), dist.get_rank()
    dev = torch.device("cuda", torch.cuda.current_device())
    ax.init(G_inter=1, G_data=world, G_intra_r=1, G_intra_c=1, G_intra_d=1)
    torch.manual_seed(5)
    layer = moe.ExpertParallelMoE(hidden, ffn, n_experts, top_k, dtype=torch.bfloat16).to(dev)
    x = (torch.randn(tokens, hidden, device=dev) * 0.5).bfloat16().requires_grad_(True)
    g = (torch.randn(tokens, hidden, device=dev) * 0.1).bfloat16()

    def step():
        layer(x).backward(g)
        x.grad = None
        for p in layer.parameters():
            p.grad = None

    def experts_batched(xin):
        return ops.linear_batched(ops.swiglu(ops.linear_batched(xin, layer.w1)), layer.w2)

    def experts_loop(xin):
        return torch.stack([ops.linear(ops.swiglu(ops.linear(xin[e], layer.w1[e])), layer.w2[e])
                            for e in range(layer.n_local)], 0)

    res = {"label": "MoE layer fwd+bwd", "tokens": tokens, "hidden": hidden, "ffn": ffn, "experts": n_experts,
           "top_k": top_k, "ranks": world, "local_experts": layer.n_local, "capacity": layer.capacity(tokens)}
    res["p2p_kernels_ms"] = round(_timed_group(step, iters, dev), 4)
    moe_kernels.DISABLED = True
    res["nccl_all_to_all_ms"] = round(_timed_group(step, iters, dev), 4)
    moe_kernels.DISABLED = False
    rows = world * layer.capacity(tokens)
    xin = (torch.randn(layer.n_local, rows, hidden, device=dev) * 0.5).bfloat16().requires_grad_(True)
    gin = (torch.randn(layer.n_local, rows, hidden, device=dev) * 0.1).bfloat16()
    for name, fn in (("experts_batched_ms", experts_batched), ("experts_loop_ms", experts_loop)):
        def run():
            fn(xin).backward(gin)
            xin.grad = None
            for p in layer.parameters():
                p.grad = None
        res[name] = round(_timed_group(run, iters, dev), 4)
    flops = 3 * 2.0 * layer.n_local * rows * hidden * ffn * 3           # fwd + dgrad + wgrad of three projections
    res["experts_tflops_batched"] = round(flops / res["experts_batched_ms"] / 1e9, 1)
    if rank == 0:
        print(json.dumps(res), flush=True)


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
    elif what == "fused_loopback_two_shot":
        bench_fused_loopback_two_shot()
    elif what in ("fused", "fused_one_shot", "ag", "rs", "grad_ar", "moe"):
        import os

        import torch.distributed as dist

        local = int(os.environ.get("LOCAL_RANK", 0))
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        if what == "fused":
            bench_fused(two_shot=True)
        elif what == "fused_one_shot":
            os.environ["AXONN_TWO_SHOT"] = "0"
            bench_fused(two_shot=False)
        elif what == "ag":
            bench_ag()
        elif what == "rs":
            bench_rs()
        elif what == "moe":
            bench_moe()
        else:
            bench_grad_ar()
        dist.destroy_process_group()
    else:
        raise SystemExit(f"unknown benchmark {what}")
