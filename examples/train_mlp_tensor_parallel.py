"""Tensor-parallel training in the three steps of the user guide, on any grid, with an elastic restart.

    python -m torch.distributed.run --nproc-per-node 4 examples/train_mlp_tensor_parallel.py \
        --G-intra-r 2 --G-intra-d 2 --steps 40 --save ckpt
    # later, on another grid (here: 2 ranks, column parallelism), continue the same run:
    python -m torch.distributed.run --nproc-per-node 2 examples/train_mlp_tensor_parallel.py \
        --G-intra-c 2 --steps 40 --resume ckpt

1. ``ax.init`` builds the process groups of the grid; 2. ``ax.create_dataloader`` hands every rank its share of
the batch; 3. ``auto_parallelize`` replaces the model's ``nn.Linear`` layers by tensor-parallel ones.  The loop
itself is ordinary PyTorch plus ``sync_gradients`` (data- and depth-parallel gradient reduction) and
``clip_grad_norm_`` (a norm over sharded parameters).  Runs on GPUs (NCCL, bf16 autocast) and on CPU ranks (gloo).

The task is synthetic (a fixed random teacher network labels random inputs), so the loss falls without any
dataset on disk.
"""

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist
import torch.nn as nn

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from axonn_b200 import axonn as ax  # noqa: E402
from axonn_b200 import checkpoint  # noqa: E402
from axonn_b200.intra_layer import (  # noqa: E402
    auto_parallelize,
    clip_grad_norm_,
    optimize_communication,
    sync_gradients,
)
from axonn_b200.optim import FusedAdamW  # noqa: E402


class TeacherDataset(torch.utils.data.Dataset):
    """``n`` random vectors labelled by a fixed random two-layer network (10 classes)."""

    def __init__(self, n=4096, width=64, seed=0):
        g = torch.Generator().manual_seed(seed)
        self.x = torch.randn(n, width, generator=g)
        w1, w2 = torch.randn(width, 128, generator=g) / 8, torch.randn(128, 10, generator=g) / 8
        self.y = (torch.tanh(self.x @ w1) @ w2).argmax(-1)

    def __len__(self):
        return len(self.x)

    def __getitem__(self, i):
        return self.x[i], self.y[i]


def main():
    ap = argparse.ArgumentParser()
    for name in ("G-data", "G-intra-r", "G-intra-c", "G-intra-d"):
        ap.add_argument("--" + name, type=int, default=None)
    ap.add_argument("--steps", type=int, default=40)
    ap.add_argument("--global-batch", type=int, default=64)
    ap.add_argument("--hidden", type=int, default=256)
    ap.add_argument("--save", default=None, help="folder for a grid-independent checkpoint after the last step")
    ap.add_argument("--resume", default=None, help="folder of a checkpoint written by --save (any grid)")
    args = ap.parse_args()

    use_cuda = torch.cuda.is_available()
    if use_cuda:
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
    dist.init_process_group(backend="nccl" if use_cuda else "gloo")
    world = dist.get_world_size()
    r, c, d = args.G_intra_r or 1, args.G_intra_c or 1, args.G_intra_d or 1
    g_data = args.G_data or world // (r * c * d)
    # ---- step 1: the grid
    ax.init(G_inter=1, G_data=g_data, G_intra_r=r, G_intra_c=c, G_intra_d=d)
    device = torch.device("cuda", torch.cuda.current_device()) if use_cuda else torch.device("cpu")

    # ---- step 2: the data
    data = TeacherDataset()
    loader = ax.create_dataloader(data, args.global_batch, micro_batch_size=args.global_batch // (g_data * d),
                                  shuffle=False)

    # ---- step 3: the model (same seed on every rank: every rank draws the full matrices and keeps its shard)
    torch.manual_seed(1)
    with auto_parallelize():
        model = nn.Sequential(nn.Linear(64, args.hidden), nn.GELU(), nn.Linear(args.hidden, args.hidden), nn.GELU(),
                              nn.Linear(args.hidden, 10)).to(device)
    opt = FusedAdamW(model.parameters(), lr=2e-3, weight_decay=0.0)
    first_step = 0
    if args.resume:
        first_step = checkpoint.load_consolidated(model, opt, args.resume, "last")["step"]

    losses, step = [], first_step
    it = iter(loader)
    for _ in range(first_step):          # the resumed run continues with the data the first run had not seen
        next(it, None)
    while step < first_step + args.steps:
        batch = next(it, None)
        if batch is None:
            loader.sampler.set_epoch(step)
            it = iter(loader)
            continue
        x, y = (t.to(device, non_blocking=True) for t in batch)
        opt.zero_grad(set_to_none=True)
        with optimize_communication(overlap_all_reduce=True, overlap_reduce_scatter=True, overlap_all_gather=True,
                                    model_object_for_overlapping_allgathers=model):
            with torch.autocast(device.type, dtype=torch.bfloat16, enabled=use_cuda):
                loss = nn.functional.cross_entropy(model(x).float(), y)
            loss.backward()
        sync_gradients(model, mean=True)
        clip_grad_norm_(model.parameters(), 1.0)
        opt.step()
        # the loss of the global batch: mean over the replicas that saw different samples
        done = loss.detach().clone()
        dist.all_reduce(done)
        losses.append(float(done) / world)
        step += 1

    if args.save:
        checkpoint.save_consolidated(model, opt, args.save, "last", extra={"step": step})
    if dist.get_rank() == 0:
        print(json.dumps({"grid": {"G_data": g_data, "r": r, "c": c, "d": d}, "first_step": first_step, "steps": step,
                          "first_loss": round(losses[0], 4), "last_loss": round(losses[-1], 4)}), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
