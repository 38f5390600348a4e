"""Less-travelled options of the tensor-parallel layers on CPU ranks, each against its torch.nn counterpart:
``skip_bias_add``, ``transpose``, a per-layer ``tensor_parallel_dims``, weight caching between forward and backward,
gradient accumulation under ``no_grad_sync`` with overlapped communication, clipping with the 1- and inf-norm,
strided / bias-skipping convolutions and embeddings with a padding index."""

import pytest
import torch

from _dist import run_distributed


def _options(rank, world, grid):
    import torch.distributed as dist

    from axonn_b200 import axonn as ax
    from axonn_b200.intra_layer import (Conv2d, Embedding, Linear, clip_grad_norm_, no_grad_sync,
                                        optimize_communication, sync_gradients)
    from axonn_b200.intra_layer.communication import _drop, _gather

    r, c, d = grid
    ax.init(G_inter=1, G_data=world // (r * c * d), G_intra_r=r, G_intra_c=c, G_intra_d=d)
    ch = ax.comm_handle
    inner, outer, depth = (ch.inner_intra_layer_parallel_group, ch.outer_intra_layer_parallel_group,
                           ch.depth_intra_layer_parallel_group)
    W = dist.group.WORLD
    torch.manual_seed(1)
    H = 16
    tol = dict(rtol=1e-4, atol=1e-6)

    # ---- skip_bias_add (easy mode): the layer returns (x W^T, full bias)
    seq = torch.nn.Linear(H, 2 * H)
    par = Linear(H, 2 * H, skip_bias_add=True)
    par.load_state_dict(seq.state_dict())
    X = torch.randn(2 * world, H)
    y, b = par(_drop(X, 0, W))
    assert torch.allclose(b, seq.bias, **tol)
    assert torch.allclose(_gather((y + b).detach(), 0, W), seq(X), **tol)

    # ---- transpose=True (expert mode): input features over the OUTER group, output over the INNER group
    seq_t = torch.nn.Linear(2 * H, H)
    par_t = Linear(2 * H, H, transpose=True, expert_mode=True)
    par_t.load_state_dict(seq_t.state_dict())
    Xt = torch.randn(2 * d * ax.config.G_data, 2 * H)
    dp = ch.data_parallel_group
    xt = _drop(_drop(_drop(Xt, 0, dp), 0, depth), 1, outer).clone().requires_grad_(True)
    yt = par_t(xt)
    full = _gather(_gather(_gather(yt.detach(), 1, inner), 0, depth), 0, dp)
    assert torch.allclose(full, seq_t(Xt), **tol), (full - seq_t(Xt)).abs().max()

    # ---- a per-layer grid: all tensor-parallel ranks on the output dimension
    tp = r * c * d
    seq_p = torch.nn.Linear(H, 4 * tp)
    par_p = Linear(H, 4 * tp, expert_mode=True, tensor_parallel_dims=(tp, 1, 1))
    par_p.load_state_dict(seq_p.state_dict())
    assert par_p.local_weight_shape == (4, H) and par_p.depth_group_size == 1
    Xp = torch.randn(3, H)
    yp = par_p(Xp)                                                  # every rank: the same rows, its 4 columns
    assert torch.allclose(_gather(yp.detach(), 1, par_p.outer_group), seq_p(Xp), **tol)

    # ---- weights cached between forward and backward, two microbatches accumulated without synchronisation
    seq_a = torch.nn.Linear(H, H)
    par_a = Linear(H, H)
    par_a.load_state_dict(seq_a.state_dict())
    Xa = [torch.randn(2 * world, H) for _ in range(2)]
    with optimize_communication(overlap_all_reduce=True, overlap_reduce_scatter=True, cache_weights=True,
                                overlap_all_gather=True, model_object_for_overlapping_allgathers=par_a):
        with no_grad_sync():
            for xa in Xa:
                par_a(_drop(xa, 0, W)).square().sum().backward()
    # no_grad_sync suppressed the data-parallel reduction: do it now, once
    sync_gradients(par_a)
    for xa in Xa:
        seq_a(xa).square().sum().backward()
    assert torch.allclose(par_a.full_tensor("weight", par_a.weight.grad), seq_a.weight.grad, rtol=1e-4, atol=1e-5)
    assert torch.allclose(par_a.full_tensor("bias", par_a.bias.grad), seq_a.bias.grad, rtol=1e-4, atol=1e-5)

    # ---- clipping with other norms
    for norm_type in (1.0, float("inf")):
        want = torch.nn.utils.clip_grad_norm_(seq_a.parameters(), 1e9, norm_type=norm_type)
        got = clip_grad_norm_(par_a.parameters(), 1e9, norm_type=norm_type)
        assert float(got) == pytest.approx(float(want), rel=1e-4), (norm_type, float(got), float(want))

    # ---- convolution: stride 2, bias returned separately
    seq_c = torch.nn.Conv2d(8, 16, 3, stride=2, padding=1)
    par_c = Conv2d(8, 16, 3, stride=2, padding=1, skip_bias_add=True)
    par_c.load_state_dict(seq_c.state_dict())
    Xc = torch.randn(2 * d, 8, 8, 8)
    yc, bc = par_c(Xc)
    assert torch.allclose(yc + bc.view(1, -1, 1, 1), seq_c(Xc), atol=1e-5)

    # ---- embedding with a padding index (row stays zero, receives no gradient)
    if c == 1:
        seq_e = torch.nn.Embedding(32, 8, padding_idx=3)
        par_e = Embedding(32, 8, padding_idx=3)
        par_e.load_state_dict(seq_e.state_dict())
        ids = torch.tensor([[3, 1, 3, 30], [0, 3, 7, 7]])
        ye = par_e(ids)
        assert torch.allclose(ye, seq_e(ids)) and float(ye[0, 0].abs().sum()) == 0.0
        ye.sum().backward()
        ge = par_e.full_tensor("weight", par_e.weight.grad) / d    # every depth rank looked up the same ids
        seq_e(ids).sum().backward()
        assert torch.allclose(ge, seq_e.weight.grad) and float(ge[3].abs().sum()) == 0.0
    return True


@pytest.mark.parametrize("grid", [(2, 2, 1), (1, 2, 2), (2, 1, 2)])
def test_layer_options_match_torch(grid):
    assert all(run_distributed(_options, 4, grid))


def _easy_trainer(rank, world, grid):
    """``Trainer`` around an auto-parallelised (easy-mode) model with a user loss function: every rank feeds its own
    shard of the batch; three AdamW steps must follow single-process training on the whole batch."""
    import torch.distributed as dist

    from axonn_b200 import axonn as ax
    from axonn_b200.intra_layer import auto_parallelize
    from axonn_b200.optim import FusedAdamW
    from axonn_b200.trainer import Trainer

    r, c, d = grid
    ax.init(G_inter=1, G_data=world // (r * c * d), G_intra_r=r, G_intra_c=c, G_intra_d=d)

    def build():
        torch.manual_seed(3)
        return torch.nn.Sequential(torch.nn.Linear(16, 32), torch.nn.GELU(), torch.nn.Linear(32, 8))

    ref = build()
    with auto_parallelize():
        par = build()
    par.load_state_dict(ref.state_dict())
    loss_fn = torch.nn.functional.cross_entropy
    tr = Trainer(par, FusedAdamW(par.parameters(), lr=1e-2, weight_decay=0.0), loss_fn=loss_fn, expert_mode=False,
                 clip_grad=1.0)
    opt = torch.optim.AdamW(ref.parameters(), lr=1e-2, weight_decay=0.0)
    g = torch.Generator().manual_seed(9)
    losses = []
    for _ in range(3):
        X, Y = torch.randn(4 * world, 16, generator=g), torch.randint(0, 8, (4 * world,), generator=g)
        mine = tr.train_step(X[rank * 4:(rank + 1) * 4], Y[rank * 4:(rank + 1) * 4])
        t = torch.tensor(mine, dtype=torch.float64)
        dist.all_reduce(t)
        opt.zero_grad()
        loss = loss_fn(ref(X), Y)
        loss.backward()
        torch.nn.utils.clip_grad_norm_(ref.parameters(), 1.0)
        opt.step()
        losses.append((float(t) / world, float(loss)))
    for got, want in losses:
        assert got == pytest.approx(want, rel=1e-4), losses
    assert torch.allclose(par[0].full_weight(), ref[0].weight, rtol=1e-3, atol=1e-5)
    assert torch.allclose(par[2].full_tensor("bias"), ref[2].bias, rtol=1e-3, atol=1e-5)
    return True


@pytest.mark.parametrize("grid", [(2, 1, 2), (1, 1, 2)])
def test_trainer_with_easy_mode_model_and_user_loss(grid):
    assert all(run_distributed(_easy_trainer, 4, grid))
