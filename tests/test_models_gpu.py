"""One-GPU training smoke of every model family through the package's kernels (child process, NCCL world of 1):
the loss falls over a few AdamW steps and no kernel reports an expired wait."""

import pytest
import torch

from _dist import run_distributed

pytestmark = pytest.mark.gpu


def _train(rank, world, family):
    from axonn_b200 import axonn as ax
    from axonn_b200.models import GPT, GPTConfig, Llama, LlamaConfig, Mixtral, MixtralConfig
    from axonn_b200.ops import _lib
    from axonn_b200.optim import FusedAdamW
    from axonn_b200.trainer import Trainer

    if family == "mixtral":
        ax.init(G_inter=1, G_data=world)
    else:
        ax.init(G_inter=1, G_data=1, G_intra_r=1, G_intra_c=1, G_intra_d=world)
    torch.manual_seed(0)
    if family == "gpt":
        cfg = GPTConfig(n_layers=2, hidden=256, n_heads=4, ffn=1024, vocab=1024, seq_len=128)
        model = GPT(cfg)
    elif family == "llama":
        cfg = LlamaConfig(n_layers=2, hidden=256, n_heads=4, n_kv_heads=2, ffn=512, vocab=1024, seq_len=128)
        model = Llama(cfg)
    else:
        cfg = MixtralConfig(n_layers=2, hidden=256, n_heads=4, n_kv_heads=2, ffn=512, n_experts=4, vocab=1024, seq_len=128)
        model = Mixtral(cfg)
    tr = Trainer(model, FusedAdamW(model.parameters(), lr=1e-3), micro_batch_size=4, clip_grad=1.0,
                 prune_keep_fraction=0.5 if family == "llama" else None)
    g = torch.Generator().manual_seed(1 + rank)
    tokens = torch.randint(0, cfg.vocab, (4, cfg.seq_len + 1), generator=g)
    losses = [tr.train_step(tokens[:, :-1].contiguous(), tokens[:, 1:].contiguous()) for _ in range(6)]
    assert _lib.device_status() == 0
    return losses


@pytest.mark.parametrize("family", ["gpt", "llama", "mixtral"])
def test_model_family_trains_on_one_gpu(family):
    losses = run_distributed(_train, 1, family, backend="nccl", timeout=300)[0]
    assert losses[-1] == losses[-1] and losses[-1] < losses[0], losses


@pytest.mark.multigpu
@pytest.mark.parametrize("family", ["llama", "mixtral"])
def test_model_family_trains_on_two_gpus(family):
    """Llama with depth-sharded weights (in-kernel weight all-gather, fused reduce-scatter, peer-memory embedding
    rows, gradient pruning) and Mixtral with expert parallelism over two ranks."""
    import os

    os.environ["NCCL_NVLS_ENABLE"] = "0"
    for losses in run_distributed(_train, 2, family, backend="nccl", timeout=300):
        assert losses[-1] == losses[-1] and losses[-1] < losses[0], losses
