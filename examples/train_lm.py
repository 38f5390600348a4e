"""Language-model training on a token file (or a synthetic stream) with tensor and data parallelism.

    python -m torch.distributed.run --nproc-per-node 4 examples/train_lm.py --G-intra-r 2 --G-intra-d 2 \
        --data corpus.txt --model small --steps 200

The counterpart of the upstream ``examples/test_lm.py`` (GPT on WikiText / Penn Treebank): ``--data`` names a file
of token ids (``.npy``, or raw ``.bin`` of uint16) or any text file, which is then modelled byte by byte; without
``--data`` a synthetic stream with learnable structure is generated.  The model is the package's tensor-parallel
GPT; ``Trainer`` runs the step (microbatches, communication overlap, gradient synchronisation, clipping,
``FusedAdamW``).  Prints one JSON line with the first and last loss and the tokens per second.
"""

import argparse
import json
import os
import sys
import time

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from axonn_b200 import axonn as ax  # noqa: E402
from axonn_b200.models import GPT, GPTConfig  # noqa: E402
from axonn_b200.optim import FusedAdamW  # noqa: E402
from axonn_b200.trainer import Trainer  # noqa: E402
from axonn_b200.utils.data import TokenWindows, load_tokens  # noqa: E402

MODELS = {
    "tiny": dict(n_layers=2, hidden=128, n_heads=4, ffn=512),
    "small": dict(n_layers=12, hidden=768, n_heads=12, ffn=3072),
    "medium": dict(n_layers=24, hidden=1024, n_heads=16, ffn=4096),
    "1.3b": dict(n_layers=24, hidden=2048, n_heads=16, ffn=8192),
}


def synthetic_stream(n, vocab, seed=0):
    """A second-order pattern with noise: token t is mostly a fixed function of the two tokens before it."""
    rng = np.random.default_rng(seed)
    table = rng.integers(0, vocab, size=(vocab, 8))
    out = np.empty(n, dtype=np.int64)
    out[:2] = rng.integers(0, vocab, size=2)
    noise = rng.random(n) < 0.1
    rand = rng.integers(0, vocab, size=n)
    for t in range(2, n):
        out[t] = rand[t] if noise[t] else table[out[t - 1], out[t - 2] % 8]
    return out


def main():
    ap = argparse.ArgumentParser()
    for name in ("G-data", "G-intra-r", "G-intra-c", "G-intra-d"):
        ap.add_argument("--" + name, type=int, default=None)
    ap.add_argument("--data", default=None)
    ap.add_argument("--model", choices=sorted(MODELS), default="tiny")
    ap.add_argument("--seq-len", type=int, default=128)
    ap.add_argument("--vocab", type=int, default=None, help="default: 256 for text files, 512 for the synthetic stream")
    ap.add_argument("--global-batch", type=int, default=16)
    ap.add_argument("--micro-batch", type=int, default=None)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--lr", type=float, default=3e-3)
    args = ap.parse_args()

    use_cuda = torch.cuda.is_available()
    if use_cuda:
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
    dist.init_process_group(backend="nccl" if use_cuda else "gloo")
    world = dist.get_world_size()
    r, c, d = args.G_intra_r or 1, args.G_intra_c or 1, args.G_intra_d or 1
    g_data = args.G_data or world // (r * c * d)
    ax.init(G_inter=1, G_data=g_data, G_intra_r=r, G_intra_c=c, G_intra_d=d)

    if args.data:
        tokens = load_tokens(args.data)
        vocab = args.vocab or (256 if tokens.dtype == np.uint8 else int(np.max(tokens)) + 1)
    else:
        vocab = args.vocab or 512
        tokens = synthetic_stream(200_000, vocab)
    vocab = -(-vocab // (8 * r * c)) * (8 * r * c)            # the vocabulary-parallel head wants whole 8-column slices
    data = TokenWindows(tokens, args.seq_len, vocab=vocab)
    per_replica = args.global_batch // (g_data * d)
    loader = ax.create_dataloader(data, args.global_batch, micro_batch_size=per_replica, shuffle=True)

    torch.manual_seed(0)
    cfg = GPTConfig(vocab=vocab, seq_len=args.seq_len, **MODELS[args.model])
    model = GPT(cfg, dtype=torch.bfloat16 if use_cuda else torch.float32)
    opt = FusedAdamW(model.parameters(), lr=args.lr, weight_decay=0.01)
    trainer = Trainer(model, opt, micro_batch_size=args.micro_batch or per_replica, clip_grad=1.0)

    losses, step, epoch = [], 0, 0
    t0 = None
    while step < args.steps:
        loader.sampler.set_epoch(epoch)
        for x, y in loader:
            if step == min(3, args.steps - 1):
                if use_cuda:
                    torch.cuda.synchronize()
                t0, timed_from = time.perf_counter(), step
            loss = torch.tensor(trainer.train_step(x, y))
            dist.all_reduce(loss)                            # replicas saw different samples: report their mean
            losses.append(float(loss) / world)
            step += 1
            if step >= args.steps:
                break
        epoch += 1
    if use_cuda:
        torch.cuda.synchronize()
    elapsed = time.perf_counter() - t0
    if dist.get_rank() == 0:
        tps = (step - timed_from) * args.global_batch * args.seq_len / max(elapsed, 1e-9)
        print(json.dumps({"model": args.model, "vocab": vocab, "grid": {"G_data": g_data, "r": r, "c": c, "d": d},
                          "steps": step, "first_loss": round(losses[0], 4), "last_loss": round(losses[-1], 4),
                          "tokens_per_s": round(tps, 1)}), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
