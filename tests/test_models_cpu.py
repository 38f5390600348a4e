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


def _generate(rank, world, family, grid):
    from axonn_b200 import axonn as ax
    from axonn_b200.models import GPT, GPTConfig, Llama, LlamaConfig, greedy_generate, parallel_argmax

    r, c, d = grid
    ax.init(G_inter=1, G_data=world // (r * c * d), G_intra_r=r, G_intra_c=c, G_intra_d=d)
    torch.manual_seed(4)
    if family == "gpt":
        model = GPT(GPTConfig(n_layers=2, hidden=64, n_heads=4, ffn=128, vocab=128, seq_len=24), dtype=torch.float32)
    else:
        model = Llama(LlamaConfig(n_layers=2, hidden=64, n_heads=4, n_kv_heads=2, ffn=128, vocab=128, seq_len=24),
                      dtype=torch.float32)
    prompt = torch.tensor([[5, 17, 99, 3], [64, 2, 2, 120]])
    out = greedy_generate(model, prompt, 6)
    assert out.shape == (2, 10) and torch.equal(out[:, :4], prompt) and model.training
    # decoding stops at the sequence length of the model, and at an end-of-sequence token
    assert greedy_generate(model, prompt, 100).shape[1] == 24
    eos = int(out[0, 5])
    stopped = greedy_generate(model, prompt, 6, eos_id=eos)
    assert bool((stopped[0, 5:] == eos).all())
    # ties go to the lowest global index, whichever rank holds it
    group = getattr(model.head, "group", None)
    tied = torch.zeros(3, model(prompt).shape[-1])
    assert parallel_argmax(tied, group).tolist() == [0, 0, 0]
    return out.tolist()


@pytest.mark.parametrize("family", ["gpt", "llama"])
def test_greedy_decoding_is_the_same_on_every_grid(family):
    ref = run_distributed(_generate, 1, family, (1, 1, 1))[0]
    for world, grid in (((2, (2, 1, 1)),) if family == "llama" else ((4, (1, 2, 2)),)):
        for got in run_distributed(_generate, world, family, grid):
            assert got == ref, (grid, got, ref)
