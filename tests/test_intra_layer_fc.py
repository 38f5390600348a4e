"""Tensor-parallel Linear == torch.nn.Linear, on CPU ranks (gloo).

Pattern of the reference's ``axonn/tests/test_intra_layer_fc.py``: build both
layers, load the sequential state dict into the parallel one, shard the input,
gather outputs / gradients, compare.  Covers every grid up to 2x2x2, easy and
expert mode, bias (including bias gradients, skipped upstream), all overlap
options, gradient clipping and full<->sharded state-dict loading.
"""

import pytest
import torch

from _dist import run_distributed


def _fc_case(rank, world, grid, expert_mode, bias, comm_opt, clip, B, H):
    import torch.distributed as dist

    from axonn_b200 import axonn as ax
    from axonn_b200.intra_layer import (Linear, clip_grad_norm_, optimize_communication, sync_gradients)
    from axonn_b200.intra_layer.communication import _drop, _gather

    r, c, d = grid
    ax.init(G_inter=1, G_data=world // (r * c * d), G_intra_r=r, G_intra_c=c, G_intra_d=d)
    ch = ax.comm_handle
    inner, outer, depth = (ch.inner_intra_layer_parallel_group, ch.outer_intra_layer_parallel_group,
                           ch.depth_intra_layer_parallel_group)
    torch.manual_seed(42)
    seq = torch.nn.Linear(H, 2 * H, bias=bias)
    par = Linear(H, 2 * H, bias=bias, expert_mode=expert_mode)
    par.load_state_dict(seq.state_dict())
    # also accept its own sharded state dict
    par.load_state_dict(par.state_dict())
    X = torch.randn(B * world, H) * 0.1
    Xs = X.clone().requires_grad_(True)
    Ys = seq(Xs)
    Gy = torch.randn_like(Ys) * 0.1
    Ys.backward(Gy)
    if clip > 0:
        torch.nn.utils.clip_grad_norm_(seq.parameters(), clip)

    dp = ch.data_parallel_group
    if expert_mode:
        # input: batch split over data then depth, features over inner; output features over outer
        xl = _drop(_drop(_drop(X, 0, dp), 0, depth), 1, inner).clone().requires_grad_(True)
        gl = _drop(_drop(_drop(Gy, 0, dp), 0, depth), 1, outer).clone()
    else:
        # pure data parallel view: every rank of the world owns a batch shard
        xl = _drop(X, 0, dist.group.WORLD).clone().requires_grad_(True)
        gl = _drop(Gy, 0, dist.group.WORLD).clone()

    with optimize_communication(overlap_all_reduce=comm_opt, overlap_reduce_scatter=comm_opt,
                                cache_weights=comm_opt, overlap_all_gather=comm_opt,
                                model_object_for_overlapping_allgathers=par):
        yl = par(xl)
        yl.backward(gl)
    sync_gradients(par, expert_mode=expert_mode)
    if clip > 0:
        clip_grad_norm_(par.parameters(), clip)

    if expert_mode:
        y = _gather(_gather(_gather(yl.detach(), 1, outer), 0, depth), 0, dp)
        gx = _gather(_gather(_gather(xl.grad, 1, inner), 0, depth), 0, dp)
    else:
        y = _gather(yl.detach(), 0, dist.group.WORLD)
        gx = _gather(xl.grad, 0, dist.group.WORLD)
    tol = dict(rtol=1e-4, atol=1e-6)
    assert torch.allclose(y, Ys.detach(), **tol), (y - Ys).abs().max()
    assert torch.allclose(gx, Xs.grad, **tol), (gx - Xs.grad).abs().max()
    gw = _gather(par.weight.grad, 0, depth).reshape(par.local_weight_shape)
    gw = _gather(_gather(gw, 1, inner), 0, outer)
    assert torch.allclose(gw, seq.weight.grad, **tol), (gw - seq.weight.grad).abs().max()
    if bias:
        gb = _gather(par.bias.grad, 0, outer)
        assert torch.allclose(gb, seq.bias.grad, **tol), (gb - seq.bias.grad).abs().max()
    assert torch.allclose(par.full_weight(), seq.weight.detach())
    return True


def _fc_suite(rank, world, cases):
    for case in cases:
        try:
            _fc_case(rank, world, *case)
        except AssertionError as e:
            raise AssertionError(f"case {case}: {e}")
    return len(cases)


GRIDS_2 = [(2, 1, 1), (1, 2, 1), (1, 1, 2)]


def test_fc_world2_all_modes():
    cases = []
    for grid in GRIDS_2:
        for expert in (False, True):
            for bias in (False, True):
                cases.append((grid, expert, bias, False, -1, 4, 64))
                cases.append((grid, expert, bias, True, 1e-3, 2, 32))
    assert run_distributed(_fc_suite, 2, cases) == [len(cases)] * 2


def test_fc_world4_grids():
    cases = []
    for grid in [(2, 2, 1), (2, 1, 2), (1, 2, 2), (4, 1, 1), (1, 1, 4), (2, 1, 1)]:
        for expert in (False, True):
            cases.append((grid, expert, True, True, -1, 2, 32))
    assert run_distributed(_fc_suite, 4, cases) == [len(cases)] * 4


@pytest.mark.slow
def test_fc_world8_2x2x2():
    cases = [((2, 2, 2), e, True, o, -1, 2, 32) for e in (False, True) for o in (False, True)]
    assert run_distributed(_fc_suite, 8, cases, timeout=600) == [len(cases)] * 8


def _mlp_config1(rank, world):
    """2-layer MLP 1024->4096->1024 (GELU), fp32, G_intra_r=2, one SGD step lr 1e-3
    against single-process torch.nn.Linear."""
    import torch.distributed as dist

    from axonn_b200 import axonn as ax
    from axonn_b200.intra_layer import Linear, sync_gradients
    from axonn_b200.intra_layer.communication import _gather

    ax.init(G_inter=1, G_data=1, G_intra_r=2, G_intra_c=1, G_intra_d=1)
    torch.manual_seed(0)
    x = torch.randn(32, 1024)
    t = torch.randn(32, 1024)
    ref = torch.nn.Sequential(torch.nn.Linear(1024, 4096), torch.nn.GELU(), torch.nn.Linear(4096, 1024))
    fc1 = Linear(1024, 4096, expert_mode=True)
    fc2 = Linear(4096, 1024, expert_mode=True, transpose=True)
    fc1.load_state_dict(ref[0].state_dict())
    fc2.load_state_dict(ref[2].state_dict())
    par = torch.nn.Sequential(fc1, torch.nn.GELU(), fc2)
    opt_ref = torch.optim.SGD(ref.parameters(), lr=1e-3)
    opt_par = torch.optim.SGD(par.parameters(), lr=1e-3)
    loss_ref = torch.nn.functional.mse_loss(ref(x), t)
    loss_ref.backward()
    opt_ref.step()
    # fc2 (transpose) reduces over the row group and adds a bias that every row
    # rank holds in full: divide its bias gradient contribution accordingly
    out = par(x)
    loss = torch.nn.functional.mse_loss(out, t)
    loss.backward()
    sync_gradients(par, expert_mode=True)
    opt_par.step()
    assert torch.allclose(loss, loss_ref, rtol=1e-5, atol=1e-7)
    assert torch.allclose(fc1.full_weight(), ref[0].weight, rtol=1e-5, atol=1e-7)
    assert torch.allclose(fc2.full_weight(), ref[2].weight, rtol=1e-5, atol=1e-7)
    outer = ax.comm_handle.outer_intra_layer_parallel_group
    assert torch.allclose(_gather(fc1.bias.detach(), 0, outer), ref[0].bias, rtol=1e-5, atol=1e-7)
    assert torch.allclose(fc2.bias.detach(), ref[2].bias, rtol=1e-5, atol=1e-7)
    return float(loss)


def test_mlp_config1_world2():
    a, b = run_distributed(_mlp_config1, 2)
    assert a == b


def _fc_uneven(rank, world, grid):
    """Easy mode with a different number of rows on every rank (the variable-size layout switches)."""
    import torch.distributed as dist

    from axonn_b200 import axonn as ax
    from axonn_b200.intra_layer import Linear, sync_gradients

    r, c, d = grid
    ax.init(G_inter=1, G_data=world // (r * c * d), G_intra_r=r, G_intra_c=c, G_intra_d=d)
    torch.manual_seed(7)
    H = 16
    seq = torch.nn.Linear(H, 2 * H)
    par = Linear(H, 2 * H)
    par.load_state_dict(seq.state_dict())
    sizes = [3 + 2 * i for i in range(world)]                 # 3, 5, 7, 9 rows
    X = torch.randn(sum(sizes), H)
    G = torch.randn(sum(sizes), 2 * H)
    lo = sum(sizes[:rank])
    x = X[lo:lo + sizes[rank]].clone().requires_grad_(True)
    for _ in range(2):                                        # the second pass uses the cached row counts
        x.grad = None
        par.zero_grad()
        y = par(x)
        y.backward(G[lo:lo + sizes[rank]])
    sync_gradients(par)
    xs = X.clone().requires_grad_(True)
    ys = seq(xs)
    ys.backward(G)
    assert y.shape == (sizes[rank], 2 * H)
    assert torch.allclose(y, ys[lo:lo + sizes[rank]], atol=1e-5), (y - ys[lo:lo + sizes[rank]]).abs().max()
    assert torch.allclose(x.grad, xs.grad[lo:lo + sizes[rank]], atol=1e-5)
    assert torch.allclose(par.full_tensor("weight", par.weight.grad), seq.weight.grad, atol=1e-4)
    assert torch.allclose(par.full_tensor("bias", par.bias.grad), seq.bias.grad, atol=1e-4)
    # a rank changes its batch size: the counts are exchanged again
    x2 = X[:sizes[rank] + 1].clone()
    assert torch.allclose(par(x2), seq(x2), atol=1e-5)
    return True


@pytest.mark.parametrize("grid", [(2, 2, 1), (1, 2, 2), (4, 1, 1)])
def test_fc_easy_mode_with_uneven_batches(grid):
    assert all(run_distributed(_fc_uneven, 4, grid))
