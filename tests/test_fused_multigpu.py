"""Fused GEMM + all-reduce over NVLink peer memory against NCCL + a plain
PyTorch fp32 reference, on 2 GPUs (child processes, NVLS off)."""

import os

import pytest
import torch

from _dist import run_distributed

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


def _gemm_ar_case(rank, world, two_shot):
    import torch.distributed as dist

    from axonn_b200.ops import _lib
    from axonn_b200.parallel import fused, symm

    dev = torch.device("cuda", rank)
    group = dist.group.WORLD
    if two_shot:
        # outputs in a peer-mapped arena: every 32-row unit is reduced by one owner and stored on all ranks
        assert symm.create_output_arena(1 << 30) is not None
    else:
        os.environ["AXONN_TWO_SHOT"] = "0"
    results = []
    for layout, (M, N, K) in [(0, (512, 512, 256)), (0, (1000, 1288, 520)), (1, (2048, 1024, 512)),
                              (0, (4096, 4096, 1024)), (1, (640, 264, 136))]:
        for rep in range(3):  # repeated calls exercise inbox parity and epochs
            g = torch.Generator(device=dev).manual_seed(17 * rank + M + rep)
            a = (torch.randn(M, K, device=dev, generator=g) * 0.5).bfloat16()
            bshape = (N, K) if layout == 0 else (K, N)
            b = (torch.randn(bshape, device=dev, generator=g) * 0.5).bfloat16()
            out = fused.gemm_all_reduce(layout, a, b, group)
            part = (a.float() @ b.float().t()) if layout == 0 else (a.float() @ b.float())
            # reference: sum of the bf16-rounded partials of both ranks (what an NCCL bf16 all-reduce adds)
            ref = part.bfloat16().float()
            dist.all_reduce(ref)
            torch.cuda.synchronize()
            status = _lib.lib().axb_device_status(rank, 1)
            err = (out.float() - ref).abs().max().item()
            scale = ref.abs().max().item()
            results.append((layout, M, N, K, rep, status, err, scale))
            # both ranks must hold identical bits
            other = out.clone()
            dist.broadcast(other, src=0)
            assert torch.equal(other, out), "ranks disagree bitwise"
            # the reduction order is fixed (rank order): the same inputs give the same bits on every run
            again = fused.gemm_all_reduce(layout, a, b, group)
            assert torch.equal(again, out), "results differ from run to run"
    # guard bytes behind every symmetric buffer are untouched: nothing wrote past an inbox or a flag array
    from axonn_b200.parallel import symm
    assert symm.verify_canaries() >= 1
    # fused bias + GELU after the reduction
    M, N, K = 768, 512, 256
    a = torch.randn(M, K, device=dev).bfloat16()
    b = torch.randn(N, K, device=dev).bfloat16()
    bias = torch.randn(N, device=dev).bfloat16()
    dist.broadcast(bias, src=0)
    from axonn_b200 import ops
    out, aux = fused.gemm_all_reduce(0, a, b, group, bias=bias, epilogue=ops.EPI_BIAS_GELU, want_aux=True)
    ref = (a.float() @ b.float().t()).bfloat16().float()
    dist.all_reduce(ref)
    z = ref + bias.float()
    gz = torch.nn.functional.gelu(z, approximate="tanh")
    torch.cuda.synchronize()
    results.append(("gelu", (aux.float() - z).abs().max().item() / z.abs().max().item(),
                    (out.float() - gz).abs().max().item() / gz.abs().max().item()))
    return results


def _gemm_rs_case(rank, world):
    import torch.distributed as dist

    from axonn_b200.ops import _lib
    from axonn_b200.parallel import fused

    dev = torch.device("cuda", rank)
    group = dist.group.WORLD
    out = []
    for (M, N, K) in [(512, 256, 1024), (2048, 1024, 4096), (4096, 2048, 512), (96 * world, 136, 264)]:
        for rep in range(2):
            g = torch.Generator(device=dev).manual_seed(31 * rank + M + rep)
            a = (torch.randn(K, M, device=dev, generator=g) * 0.5).bfloat16()   # dY  [tokens, out]
            b = (torch.randn(K, N, device=dev, generator=g) * 0.5).bfloat16()   # X   [tokens, in]
            assert fused.reduce_scatter_usable(group, a, b, M)
            shard = fused.gemm_reduce_scatter(2, a, b, group)
            full = (a.float().t() @ b.float()).bfloat16().float()
            dist.all_reduce(full)
            R = M // world
            want = full[rank * R:(rank + 1) * R]
            torch.cuda.synchronize()
            status = _lib.lib().axb_device_status(rank, 1)
            err = (shard.float() - want).abs().max().item()
            out.append((M, N, K, status, err, want.abs().max().item()))
            # accumulate into an fp32 buffer
            acc = torch.ones(R, N, device=dev)
            fused.gemm_reduce_scatter(2, a, b, group, out=acc, accumulate=True)
            torch.cuda.synchronize()
            err2 = (acc - (want + 1)).abs().max().item()
            out.append((M, N, K, _lib.lib().axb_device_status(rank, 1), err2, want.abs().max().item()))
    return out


@pytest.mark.parametrize("world", [2, 4, 8])
def test_gemm_reduce_scatter(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    for per_rank in run_distributed(_gemm_rs_case, world, backend="nccl", timeout=300):
        for M, N, K, status, err, scale in per_rank:
            assert status == 0
            assert err <= 1.6e-2 * scale + 1e-3, (M, N, K, err, scale)


def _grad_ar_case(rank, world, mode):
    import torch.distributed as dist

    from axonn_b200 import ops
    from axonn_b200.ops import _lib

    # "fused": one kernel straight from / to the gradient tensors; "bucket": pack -> two-shot -> unpack;
    # "nvls": the bucket form with the reduction inside the NVSwitch (falls back to two-shot without multicast)
    os.environ["AXONN_GRAD_AR"] = mode
    dev = torch.device("cuda", rank)
    out = []
    for dtype in (torch.bfloat16, torch.float32):
        for rep in range(3):
            g = torch.Generator(device=dev).manual_seed(5 * rank + rep)
            grads = [torch.randn(n, device=dev, generator=g).to(dtype) for n in (1000, 7, 123457, 2048 * 513)]
            ref = [t.float().clone() for t in grads]
            for t in ref:
                dist.all_reduce(t)
            ops.all_reduce_bucketed_(grads, dist.group.WORLD, scale=0.5)
            torch.cuda.synchronize()
            status = _lib.lib().axb_device_status(rank, 1)
            tol = 2e-2 if dtype == torch.bfloat16 else 1e-6
            err = max(((a.float() - 0.5 * b).abs().max() / (b.abs().max() + 1e-9)).item() for a, b in zip(grads, ref))
            same = []
            for a in grads:
                o = a.clone()
                dist.broadcast(o, src=0)
                same.append(bool(torch.equal(o, a)))
            out.append((str(dtype), status, err, tol, all(same)))
    return out


@pytest.mark.parametrize("world,mode", [(2, "fused"), (2, "bucket"), (2, "nvls"), (4, "fused"), (8, "fused"), (8, "nvls")])
def test_gradient_all_reduce(world, mode):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    for per_rank in run_distributed(_grad_ar_case, world, mode, backend="nccl", timeout=300):
        for name, status, err, tol, same in per_rank:
            assert status == 0 and err <= tol and same, (name, status, err)


def _ag_gemm_case(rank, world):
    import torch.distributed as dist

    from axonn_b200.ops import _lib
    from axonn_b200.parallel import fused

    dev = torch.device("cuda", rank)
    group = dist.group.WORLD
    out = []
    for layout, (M, out_l, in_l) in [(0, (1024, 256 * world, 256)), (0, (4096, 1024 * world, 1024)),
                                     (1, (2048, 512 * world, 512)), (1, (512, 128 * world, 136)),
                                     (0, (640, 128 * world, 72))]:
        for rep in range(3):
            g = torch.Generator(device=dev).manual_seed(1000 + rep + out_l)       # same full weight on all ranks
            W = (torch.randn(out_l, in_l, device=dev, generator=g) * 0.3).bfloat16()
            R = out_l // world
            shard = W[rank * R:(rank + 1) * R].reshape(-1).clone()
            ga = torch.Generator(device=dev).manual_seed(7 * rank + rep)
            a = (torch.randn(M, in_l if layout == 0 else out_l, device=dev, generator=ga) * 0.5).bfloat16()
            assert fused.all_gather_usable(group, a, shard, (out_l, in_l), layout)
            y, Wg = fused.all_gather_gemm(layout, a, shard, group, (out_l, in_l))
            torch.cuda.synchronize()
            status = _lib.lib().axb_device_status(rank, 1)
            ref = a.float() @ (W.float().t() if layout == 0 else W.float())
            err = (y.float() - ref).abs().max().item() / ref.abs().max().item()
            out.append((layout, M, out_l, in_l, status, err, bool(torch.equal(Wg, W))))
    # all-gather over one group combined with the all-reduce epilogue over the same ranks
    W = (torch.randn(256 * world, 256, device=dev, generator=torch.Generator(device=dev).manual_seed(3)) * 0.3).bfloat16()
    shard = W[rank * 256:(rank + 1) * 256].reshape(-1).clone()
    a = torch.randn(1024, 256, device=dev).bfloat16()
    y, _ = fused.all_gather_gemm(0, a, shard, group, (256 * world, 256), ar_group=group)
    ref = (a.float() @ W.float().t()).bfloat16().float()
    dist.all_reduce(ref)
    torch.cuda.synchronize()
    out.append((9, 0, 0, 0, _lib.lib().axb_device_status(rank, 1),
                (y.float() - ref).abs().max().item() / ref.abs().max().item(), True))
    return out


@pytest.mark.parametrize("world", [2, 4, 8])
def test_all_gather_gemm(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    for per_rank in run_distributed(_ag_gemm_case, world, backend="nccl", timeout=300):
        for layout, M, out_l, in_l, status, err, same in per_rank:
            assert status == 0, (layout, M, out_l, in_l, status)
            assert err < 1.6e-2 and same, (layout, M, out_l, in_l, err, same)


@pytest.mark.parametrize("world,two_shot", [(2, False), (2, True), (4, False), (4, True), (8, True)])
def test_gemm_all_reduce(world, two_shot):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    res = run_distributed(_gemm_ar_case, world, two_shot, backend="nccl", timeout=300)
    for per_rank in res:
        for r in per_rank[:-1]:
            layout, M, N, K, rep, status, err, scale = r
            assert status == 0, f"kernel reported an expired wait: {r}"
            assert err <= 1.6e-2 * scale, f"{r}"
        _, e1, e2 = per_rank[-1]
        assert e1 < 2e-2 and e2 < 2e-2


def _moe_case(rank, world):
    import torch.distributed as dist

    from axonn_b200 import axonn as ax
    from axonn_b200.ops import _lib
    from axonn_b200.parallel.moe import ExpertParallelMoE

    ax.init(G_inter=1, G_data=world)
    dev = torch.device("cuda", rank)
    torch.manual_seed(5)
    layer = ExpertParallelMoE(hidden=256, ffn=512, n_experts=4, top_k=2, capacity_factor=1.0, dtype=torch.bfloat16)
    g = torch.Generator(device=dev).manual_seed(100 + rank)
    outs = []
    for it in range(3):
        x = (torch.randn(4, 64, 256, device=dev, generator=g)).bfloat16().requires_grad_(True)
        gy = torch.randn(4, 64, 256, device=dev, generator=g).bfloat16()
        res = {}
        for mode in ("nccl", "fused"):
            os.environ["AXONN_BACKEND"] = mode
            for p in layer.parameters():
                p.grad = None
            x.grad = None
            y = layer(x)
            y.backward(gy)
            res[mode] = (y.detach().float(), x.grad.float().clone(), layer.w1.grad.float().clone(),
                         layer.router.grad.float().clone(), float(layer.last_drop_fraction))
        torch.cuda.synchronize()
        status = _lib.lib().axb_device_status(rank, 1)
        errs = [((a - b).abs().max() / (b.abs().max() + 1e-6)).item() for a, b in zip(res["fused"][:4], res["nccl"][:4])]
        outs.append((status, errs, res["fused"][4]))
    os.environ["AXONN_BACKEND"] = "fused"
    return outs


def test_moe_peer_memory_exchange_matches_all_to_all():
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    res = run_distributed(_moe_case, 2, backend="nccl", timeout=300)
    for per_rank in res:
        for status, errs, drop in per_rank:
            assert status == 0
            assert max(errs) < 3e-2, errs
            assert drop > 0.0  # capacity factor 1.0 with random routing drops some assignments
