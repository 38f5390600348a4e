"""Model-level equivalence across grids on CPU ranks: the tiny GPT and Llama
models must produce the same loss and the same updated weights on one rank and
on a 2x2x2 grid (same seed => same full matrices => same function)."""

import pytest
import torch

from _dist import run_distributed


def _train(rank, world, grid, family, steps):
    from axonn_b200 import axonn as ax
    from axonn_b200.models import GPT, GPTConfig, Llama, LlamaConfig
    from axonn_b200.optim import FusedAdamW
    from axonn_b200.trainer import Trainer, num_replicas, replica_index

    r, c, d = grid
    ax.init(G_inter=1, G_data=world // (r * c * d), G_intra_r=r, G_intra_c=c, G_intra_d=d)
    torch.manual_seed(1234)
    if family == "gpt":
        cfg = GPTConfig.tiny()
        model = GPT(cfg, dtype=torch.float32)
    else:
        cfg = LlamaConfig.tiny()
        model = Llama(cfg, dtype=torch.float32)
    opt = FusedAdamW(model.parameters(), lr=2e-3, weight_decay=0.0)
    tr = Trainer(model, opt, micro_batch_size=2, clip_grad=1.0)
    g = torch.Generator().manual_seed(7)
    B = 8
    losses = []
    tokens = torch.randint(0, cfg.vocab, (B, cfg.seq_len + 1), generator=g)
    for _ in range(steps):
        per = B // num_replicas()
        mine = tokens[replica_index() * per:(replica_index() + 1) * per]
        losses.append(tr.train_step(mine[:, :-1].contiguous(), mine[:, 1:].contiguous()))
    # average the per-replica losses (each replica saw a different slice)
    import torch.distributed as dist
    t = torch.tensor(losses, dtype=torch.float64)
    dist.all_reduce(t)
    w = model.blocks[0].mlp.fc1.full_weight()
    return (t / world).tolist(), float(w.double().pow(2).sum())


@pytest.mark.parametrize("family", ["gpt", "llama"])
def test_tiny_model_same_on_1_and_8_ranks(family):
    ref_losses, ref_w = run_distributed(_train, 1, (1, 1, 1), family, 3)[0]
    out = run_distributed(_train, 8, (2, 2, 2), family, 3, timeout=600)
    for losses, w in out:
        assert losses == pytest.approx(ref_losses, rel=2e-4)
        assert w == pytest.approx(ref_w, rel=1e-4)
    assert ref_losses[-1] < ref_losses[0]
