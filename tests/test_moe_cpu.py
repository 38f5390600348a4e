"""Expert-parallel MoE on CPU ranks: with a capacity large enough to drop
nothing, 4 expert-parallel ranks must reproduce the single-rank layer (same
seed => same experts) in output, input gradient and expert gradients."""

import torch

from _dist import run_distributed


def _moe(rank, world, ep):
    import torch.distributed as dist

    from axonn_b200 import axonn as ax
    from axonn_b200.intra_layer import sync_gradients
    from axonn_b200.parallel.moe import ExpertParallelMoE

    ax.init(G_inter=1, G_data=world)
    torch.manual_seed(5)
    layer = ExpertParallelMoE(hidden=32, ffn=64, n_experts=4, top_k=2, capacity_factor=4.0, dtype=torch.float32)
    g = torch.Generator().manual_seed(11)
    X = torch.randn(4, 8, 32, generator=g)          # 4 "ranks worth" of tokens
    G = torch.randn(4, 8, 32, generator=g)
    per = 4 // world
    x = X[rank * per:(rank + 1) * per].clone().requires_grad_(True)
    y = layer(x)
    (y * G[rank * per:(rank + 1) * per]).sum().backward()
    assert float(layer.last_drop_fraction) == 0.0
    sync_gradients(layer, expert_mode=True)  # router is replicated: summed over the data group
    # gather everything for comparison
    ys = [torch.zeros_like(y) for _ in range(world)]
    dist.all_gather(ys, y.detach())
    gxs = [torch.zeros_like(x) for _ in range(world)]
    dist.all_gather(gxs, x.grad)
    w1s = [torch.zeros_like(layer.w1.grad) for _ in range(world)]
    dist.all_gather(w1s, layer.w1.grad)
    return (torch.cat(ys).numpy(), torch.cat(gxs).numpy(), torch.cat(w1s).numpy(), layer.router.grad.numpy(),
            float(layer.last_aux_loss))


def test_expert_parallel_matches_single_rank():
    import numpy as np

    ref = run_distributed(_moe, 1, 1)[0]
    out = run_distributed(_moe, 4, 4)
    for r in out:
        for a, b in zip(r[:4], ref[:4]):
            assert np.allclose(a, b, rtol=1e-4, atol=1e-5), np.abs(a - b).max()


def test_router_capacity_and_aux_loss():
    from axonn_b200.parallel.moe import route_top_k

    torch.manual_seed(0)
    logits = torch.randn(64, 8)
    idx, gate, slot, keep, aux = route_top_k(logits, 2, capacity=4)
    assert torch.allclose(gate.sum(-1), torch.ones(64))
    # no two kept assignments share a slot of the same expert
    pairs = set()
    for t in range(64):
        for j in range(2):
            if keep[t, j]:
                key = (int(idx[t, j]), int(slot[t, j]))
                assert key not in pairs and slot[t, j] < 4
                pairs.add(key)
    assert len(pairs) <= 8 * 4
    # perfectly uniform routing gives aux == 1
    u = torch.zeros(8, 8)
    for i in range(8):
        u[i, i] = 10.0
    _, _, _, _, aux_u = route_top_k(u, 1, capacity=8)
    assert abs(float(aux_u) - 1.0) < 0.05


def _moe_easy_sync(rank, world):
    """Easy-mode ``sync_gradients`` with expert parallelism over the data group: every rank's expert
    gradients keep their own values (scaled by 1/world), the replicated router's are summed."""
    from axonn_b200 import axonn as ax
    from axonn_b200.intra_layer import sync_gradients
    from axonn_b200.parallel.moe import ExpertParallelMoE

    ax.init(G_inter=1, G_data=world)
    torch.manual_seed(5)
    layer = ExpertParallelMoE(hidden=32, ffn=64, n_experts=4, top_k=2, capacity_factor=4.0, dtype=torch.float32)
    g = torch.Generator().manual_seed(20 + rank)
    x = torch.randn(2, 8, 32, generator=g, requires_grad=True)
    layer(x).sum().backward()
    w1_before = layer.w1.grad.clone()
    router_before = layer.router.grad.clone()
    sync_gradients(layer, mean=True, expert_mode=False)
    import torch.distributed as dist

    rsum = router_before.clone()
    dist.all_reduce(rsum)
    return (torch.allclose(layer.w1.grad, w1_before / world, atol=1e-6),
            torch.allclose(layer.router.grad, rsum / world, atol=1e-6))


def test_easy_mode_sync_leaves_expert_gradients_unmixed():
    for ok_expert, ok_router in run_distributed(_moe_easy_sync, 2):
        assert ok_expert and ok_router



def _routing_stats_case(rank, world):
    from axonn_b200 import axonn as ax
    from axonn_b200.parallel.moe import ExpertParallelMoE

    ax.init(G_inter=1, G_data=world)
    torch.manual_seed(2)
    layer = ExpertParallelMoE(hidden=32, ffn=64, n_experts=4, top_k=2, capacity_factor=0.5, dtype=torch.float32)
    layer(torch.randn(3, 16, 32))
    a, d = layer.last_assignments_per_expert, layer.last_dropped_per_expert
    return (int(a.sum()), float(d.sum()), float(layer.last_drop_fraction) * 48 * 2)


def test_routing_statistics_add_up():
    """Per-expert assignment and drop counts of the last forward: they sum to tokens * top_k and to the dropped
    assignments that the drop fraction reports."""
    total, dropped, from_fraction = run_distributed(_routing_stats_case, 1)[0]
    assert total == 96
    assert dropped > 0 and abs(dropped - from_fraction) < 1e-3


def _moe_consolidated(rank, world, folder, phase):
    from axonn_b200 import axonn as ax
    from axonn_b200 import checkpoint
    from axonn_b200.optim import FusedAdamW
    from axonn_b200.parallel.moe import ExpertParallelMoE

    ax.init(G_inter=1, G_data=world)
    torch.manual_seed(5 if phase == "save" else 6)  # the loading run starts from other weights
    layer = ExpertParallelMoE(hidden=32, ffn=64, n_experts=4, top_k=2, capacity_factor=4.0, dtype=torch.float32)
    opt = FusedAdamW(layer.parameters(), lr=1e-2, weight_decay=0.0)
    g = torch.Generator().manual_seed(11)
    X = torch.randn(4, 8, 32, generator=g)
    if phase == "save":
        per = 4 // world
        layer(X[rank * per:(rank + 1) * per]).square().sum().backward()
        opt.step()
        checkpoint.save_consolidated(layer, opt, folder, "moe")
    else:
        checkpoint.load_consolidated(layer, opt, folder, "moe")
    st = opt.state[layer.w1]
    return (layer.full_tensor("w1").numpy(), layer.full_tensor("w2").numpy(), layer.router.detach().numpy(),
            layer.full_tensor("w1", st["exp_avg"]).numpy(), int(st["step"]))


def test_expert_parallel_state_moves_between_group_sizes(tmp_path):
    """Experts and their optimizer moments saved by 4 expert-parallel ranks arrive unchanged in 1 and 2 ranks."""
    import numpy as np

    folder = str(tmp_path)
    saved = run_distributed(_moe_consolidated, 4, folder, "save")[0]
    assert np.abs(saved[3]).max() > 0 and saved[4] == 1
    for world in (1, 2):
        for got in run_distributed(_moe_consolidated, world, folder, "load"):
            for a, b in zip(got[:4], saved[:4]):
                assert np.array_equal(a, b)
            assert got[4] == 1
