"""Tensor-parallel layers on GPUs (child processes over NCCL, NVLS off): the equivalence pattern of
``tests/test_intra_layer_fc.py`` - parallel layer == ``torch.nn.Linear`` / ``torch.nn.Embedding`` in forward
output, input gradient, reassembled weight gradient and bias gradient - with the fused kernels on the
default path (GEMM + all-reduce, weight all-gather inside the GEMM, weight-gradient GEMM + reduce-scatter,
row all-to-all of the easy mode, peer-memory embedding rows), for worlds of 2, 4 and 8 GPUs.  fp32 layers and
widths that the tensor-core kernels do not take must fall back to the library path and stay correct."""

import os

import pytest
import torch

from _dist import run_distributed

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


def _fc_case(rank, world, grid, expert_mode, bias, dtype_name, B, H, O):
    import torch.distributed as dist

    from axonn_b200 import axonn as ax
    from axonn_b200.intra_layer import Linear, optimize_communication, sync_gradients
    from axonn_b200.intra_layer.communication import _drop, _gather
    from axonn_b200.ops import _lib

    dtype = getattr(torch, dtype_name)
    dev = torch.device("cuda", rank)
    r, c, d = grid
    ax.init(G_inter=1, G_data=world // (r * c * d), G_intra_r=r, G_intra_c=c, G_intra_d=d)
    ch = ax.comm_handle
    inner, outer, depth = (ch.inner_intra_layer_parallel_group, ch.outer_intra_layer_parallel_group,
                           ch.depth_intra_layer_parallel_group)
    torch.manual_seed(42)
    seq = torch.nn.Linear(H, O, bias=bias, device=dev)          # fp32 reference of the same layer
    with torch.no_grad():
        seq.weight.copy_(seq.weight.to(dtype).float())           # representable in the layer's dtype
        if bias:
            seq.bias.copy_((torch.randn(O, device=dev) * 0.1).to(dtype).float())
    par = Linear(H, O, bias=bias, expert_mode=expert_mode, dtype=dtype).to(dev)
    par.load_state_dict(seq.state_dict())
    X = (torch.randn(B * world, H, device=dev) * 0.5).to(dtype).float()
    Xs = X.clone().requires_grad_(True)
    Ys = seq(Xs)
    Gy = (torch.randn_like(Ys) * 0.5).to(dtype).float()
    Ys.backward(Gy)

    dp = ch.data_parallel_group
    if expert_mode:
        xl = _drop(_drop(_drop(X, 0, dp), 0, depth), 1, inner).to(dtype).clone().requires_grad_(True)
        gl = _drop(_drop(_drop(Gy, 0, dp), 0, depth), 1, outer).to(dtype).clone()
    else:
        xl = _drop(X, 0, dist.group.WORLD).to(dtype).clone().requires_grad_(True)
        gl = _drop(Gy, 0, dist.group.WORLD).to(dtype).clone()
    with optimize_communication(overlap_all_reduce=True, overlap_reduce_scatter=True, cache_weights=False,
                                overlap_all_gather=False, model_object_for_overlapping_allgathers=par):
        yl = par(xl)
        yl.backward(gl)
    sync_gradients(par, expert_mode=expert_mode)
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    if expert_mode:
        y = _gather(_gather(_gather(yl.detach(), 1, outer), 0, depth), 0, dp)
        gx = _gather(_gather(_gather(xl.grad, 1, inner), 0, depth), 0, dp)
    else:
        y = _gather(yl.detach(), 0, dist.group.WORLD)
        gx = _gather(xl.grad, 0, dist.group.WORLD)
    rel = 2e-2 if dtype != torch.float32 else 2e-3     # fp32 GEMMs of the library path may run in TF32

    def close(a, b, what):
        err = (a.float() - b.float()).abs().max().item()
        assert err <= rel * b.abs().max().item() + 1e-5, (what, err, b.abs().max().item())

    close(y, Ys.detach(), "forward")
    close(gx, Xs.grad, "input gradient")
    gw = _gather(par.weight.grad, 0, depth).reshape(par.local_weight_shape)
    gw = _gather(_gather(gw, 1, inner), 0, outer)
    close(gw, seq.weight.grad, "weight gradient")
    if bias:
        close(_gather(par.bias.grad, 0, outer), seq.bias.grad, "bias gradient")
    return True


def _fc_suite(rank, world, cases):
    os.environ["AXONN_SYMM_ARENA_GB"] = "1"
    for case in cases:
        try:
            _fc_case(rank, world, *case)
        except AssertionError as e:
            raise AssertionError(f"case {case}: {e}")
    return len(cases)


def _grids(world):
    if world == 2:
        return [(2, 1, 1), (1, 2, 1), (1, 1, 2)]
    if world == 4:
        return [(2, 2, 1), (2, 1, 2), (1, 2, 2), (4, 1, 1), (1, 1, 4)]
    return [(2, 2, 2), (1, 1, 8), (4, 2, 1)]


@pytest.mark.parametrize("world", [2, 4, 8])
def test_linear_matches_nn_linear_on_gpus(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    cases = []
    for grid in _grids(world):
        for expert in (True, False):
            cases.append((grid, expert, True, "bfloat16", 64, 1024, 2048))   # fused kernels
        cases.append((grid, True, True, "float32", 16, 256, 512))            # fp32: library path
        # widths the kernels refuse or barely take
        cases.append((grid, True, False, "bfloat16", 16, 8 * 17 * world, 8 * 9 * world))
    cases.append((_grids(world)[0], True, True, "float32", 8, 72 * world, 36 * world))   # local width not a multiple of 8
    assert run_distributed(_fc_suite, world, cases, backend="nccl", timeout=600) == [len(cases)] * world


def _embedding_case(rank, world):
    import torch.distributed as dist

    from axonn_b200 import axonn as ax
    from axonn_b200.intra_layer import Embedding, sync_gradients
    from axonn_b200.intra_layer.communication import _gather
    from axonn_b200.ops import _lib

    dev = torch.device("cuda", rank)
    ax.init(G_inter=1, G_data=1, G_intra_r=1, G_intra_c=1, G_intra_d=world)
    depth = ax.comm_handle.depth_intra_layer_parallel_group
    out = []
    for V, H, T in [(1024, 256, 512), (50304 // 8 * 8, 512, 2048)]:
        if V % world:
            continue
        torch.manual_seed(3)
        seq = torch.nn.Embedding(V, H, device=dev)
        with torch.no_grad():
            seq.weight.copy_(seq.weight.bfloat16().float())
        res = {}
        for mode in ("1", "0"):
            os.environ["AXONN_EMBEDDING_P2P"] = mode
            par = Embedding(V, H, expert_mode=True, dtype=torch.bfloat16).to(dev)
            par.load_state_dict(seq.state_dict())
            g = torch.Generator(device=dev).manual_seed(10 + rank)
            ids = torch.randint(0, V, (4, T // 4), device=dev, generator=g)
            gy = torch.randn(4, T // 4, H, device=dev, generator=g).bfloat16()
            y = par(ids)
            y.backward(gy)
            sync_gradients(par, expert_mode=True)
            torch.cuda.synchronize()
            gw = _gather(par.weight.grad, 0, depth).reshape(V, H).float()
            res[mode] = (y.detach().float(), gw)
        # reference: all ranks' tokens contribute to the table gradient
        ys = seq(ids)
        ref_g = torch.zeros(V, H, device=dev)
        ref_g.index_add_(0, ids.reshape(-1), gy.reshape(-1, H).float())
        dist.all_reduce(ref_g)
        st = _lib.device_status()
        e_fwd = (res["1"][0] - ys.detach()).abs().max().item()
        e_bwd = (res["1"][1] - ref_g).abs().max().item() / ref_g.abs().max().item()
        e_old = (res["0"][1] - ref_g).abs().max().item() / ref_g.abs().max().item()
        out.append((V, H, st, e_fwd, e_bwd, e_old))
    os.environ["AXONN_EMBEDDING_P2P"] = "1"
    return out


@pytest.mark.parametrize("world", [2, 8])
def test_embedding_rows_over_peer_memory(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    for per_rank in run_distributed(_embedding_case, world, backend="nccl", timeout=300):
        assert per_rank
        for V, H, st, e_fwd, e_bwd, e_old in per_rank:
            assert st == 0
            assert e_fwd == 0.0, (V, H, e_fwd)          # a row fetch is exact
            assert e_bwd < 2e-2, (V, H, e_bwd, e_old)   # fp32 atomics, bf16 result
