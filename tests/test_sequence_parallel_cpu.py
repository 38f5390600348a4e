"""Sequence parallelism (all-to-all attention over the data-parallel group) on CPU ranks: every rank holds a slice of
each sequence; the mean of the ranks' losses and the synchronised gradients must equal those of one process that
sees whole sequences.  Also together with row tensor parallelism."""

import pytest
import torch

from _dist import run_cached, run_distributed


def _exchange_roundtrip(rank, world):
    import torch.distributed as dist

    from axonn_b200 import axonn as ax
    from axonn_b200.parallel.sequence import seq_all_to_all

    ax.init(G_inter=1, G_data=world)
    g = dist.group.WORLD
    full = torch.arange(2 * 8 * 4 * 3, dtype=torch.float32).reshape(2, 8, 4, 3)      # [B, S, heads, D]
    per = 8 // world
    mine = full[:, rank * per:(rank + 1) * per].clone().requires_grad_(True)         # my slice of the sequence
    heads = seq_all_to_all(mine, g, scatter_dim=2, gather_dim=1)                     # whole sequence, my heads
    hp = 4 // world
    assert torch.equal(heads, full[:, :, rank * hp:(rank + 1) * hp])
    back = seq_all_to_all(heads, g, scatter_dim=1, gather_dim=2)
    assert torch.equal(back, mine)
    (back * (rank + 1)).sum().backward()                                             # gradient comes back through both
    assert torch.equal(mine.grad, torch.full_like(mine, float(rank + 1)))
    return True


@pytest.mark.parametrize("world", [2, 4])
def test_sequence_head_exchange_is_its_own_inverse(world):
    assert all(run_distributed(_exchange_roundtrip, world))


def _lm(rank, world, family, r, sp):
    import torch.distributed as dist

    from axonn_b200 import axonn as ax
    from axonn_b200.intra_layer import sync_gradients
    from axonn_b200.models import GPT, GPTConfig, Llama, LlamaConfig
    from axonn_b200.parallel.sequence import enable_sequence_parallel, shard_sequence

    ax.init(G_inter=1, G_data=sp, G_intra_r=r)
    torch.manual_seed(2)
    if family == "gpt":
        cfg = GPTConfig(n_layers=2, hidden=64, n_heads=4, ffn=128, vocab=128, seq_len=32)
        model = GPT(cfg, dtype=torch.float32)
    else:
        cfg = LlamaConfig(n_layers=2, hidden=64, n_heads=8, n_kv_heads=4, ffn=128, vocab=128, seq_len=32)
        model = Llama(cfg, dtype=torch.float32)
    g = torch.Generator().manual_seed(5)
    data = torch.randint(0, cfg.vocab, (3, cfg.seq_len + 1), generator=g)
    x, y = data[:, :-1].contiguous(), data[:, 1:].contiguous()
    if sp > 1:
        enable_sequence_parallel(model)
        x, y = shard_sequence(x), shard_sequence(y)
        assert x.shape == (3, cfg.seq_len // sp)
    loss = model(x, y)
    loss.backward()
    sync_gradients(model, mean=True, expert_mode=True)
    total = loss.detach().clone()
    dist.all_reduce(total, group=ax.comm_handle.data_parallel_group)
    # full (grid-independent) gradients of a few parameters of different kinds
    blk = model.blocks[1]
    picks = {"qkv": blk.attn.qkv.full_tensor("weight", blk.attn.qkv.weight.grad),
             "fc2": blk.mlp.fc2.full_tensor("weight", blk.mlp.fc2.weight.grad),
             "emb": model.tok_emb.full_tensor("weight", model.tok_emb.weight.grad),
             "norm": blk.norm1.full_tensor("weight", blk.norm1.weight.grad)}
    if family == "gpt":
        picks["pos"] = model.pos_emb.full_tensor("weight", model.pos_emb.weight.grad)
    return float(total) / sp, {k: v.numpy() for k, v in picks.items()}


@pytest.mark.parametrize("family,r,sp", [("gpt", 1, 2), ("llama", 1, 4), ("llama", 2, 2)])
def test_sequence_parallel_model_matches_whole_sequences(family, r, sp):
    import numpy as np

    ref_loss, ref_grads = run_cached(_lm, 1, family, 1, 1)[0]
    for loss, grads in run_distributed(_lm, r * sp, family, r, sp):
        assert loss == pytest.approx(ref_loss, rel=1e-5)
        for k, v in grads.items():
            assert np.allclose(v, ref_grads[k], rtol=2e-4, atol=1e-6), (k, np.abs(v - ref_grads[k]).max())


def _bad_head_count(rank, world):
    from axonn_b200 import axonn as ax
    from axonn_b200.models import Llama, LlamaConfig
    from axonn_b200.parallel.sequence import enable_sequence_parallel

    ax.init(G_inter=1, G_data=world)
    model = Llama(LlamaConfig(n_layers=1, hidden=96, n_heads=6, n_kv_heads=3, ffn=128, vocab=128, seq_len=32),
                  dtype=torch.float32)
    try:
        enable_sequence_parallel(model)
    except ValueError as e:
        return str(e)
    return "accepted"


def test_head_count_must_split_over_the_sequence_group():
    assert all("do not split over 2" in m for m in run_distributed(_bad_head_count, 2))
