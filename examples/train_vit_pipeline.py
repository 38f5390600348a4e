"""A small vision transformer trained with pipeline x data parallelism through ``AxoNN_Inter_Layer_Engine``.

    G_inter=2 G_data=2 python -m torch.distributed.run --nproc-per-node 4 examples/train_vit_pipeline.py

Same knobs as the upstream project's ViT check (environment variables ``G_inter``, ``G_data``, ``batch_size``,
``micro_batch_size``, ``epochs``; upstream ``axonn/tests/test_vit.py:21-25``), without its MNIST download: the
images are ten fixed 28x28 prototypes plus noise, so a run needs no dataset and the loss still falls to a few
hundredths within one epoch.  Each pipeline stage builds only its own layers; the engine moves activations and
gradients between the stages, microbatch by microbatch, and reduces gradients over the data-parallel group.
Runs on GPUs (NCCL point-to-point, bf16) and on CPU ranks (gloo, fp32).  The script exits non-zero when the
final loss is not below ``--target-loss``.
"""

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from axonn_b200 import axonn as ax  # noqa: E402
from axonn_b200.inter_layer import AxoNN_Inter_Layer_Engine  # noqa: E402
from axonn_b200.models import DistributedViT  # noqa: E402


class PrototypeDigits(torch.utils.data.Dataset):
    """``n`` images: one of ten fixed random 28x28 prototypes plus Gaussian noise; the label is the prototype."""

    def __init__(self, n=2048, noise=0.5, seed=0):
        g = torch.Generator().manual_seed(seed)
        protos = torch.randn(10, 1, 28, 28, generator=g)
        self.y = torch.randint(0, 10, (n,), generator=g)
        self.x = protos[self.y] + noise * torch.randn(n, 1, 28, 28, generator=g)

    def __len__(self):
        return len(self.y)

    def __getitem__(self, i):
        return self.x[i], self.y[i]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--target-loss", type=float, default=0.1)
    ap.add_argument("--samples", type=int, default=2048)
    args = ap.parse_args()
    G_inter, G_data = int(os.environ.get("G_inter", 2)), int(os.environ.get("G_data", 1))
    bs, mbs = int(os.environ.get("batch_size", 64)), int(os.environ.get("micro_batch_size", 8))
    epochs = int(os.environ.get("epochs", 1))

    use_cuda = torch.cuda.is_available()
    if use_cuda:
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
    dist.init_process_group(backend="nccl" if use_cuda else "gloo")
    assert dist.get_world_size() == G_inter * G_data, "launch G_inter * G_data processes"
    ax.init(G_inter=G_inter, G_data=G_data)
    device = torch.device("cuda", torch.cuda.current_device()) if use_cuda else torch.device("cpu")

    torch.manual_seed(7 + ax.config.inter_layer_parallel_rank)    # data-parallel replicas of a stage start equal
    model = DistributedViT(image_size=28, patch_size=4, num_classes=10, dim=128, depth=6 if G_inter in (1, 2, 3, 6)
                           else 2 * G_inter, heads=8, mlp_dim=256, channels=1).to(device)
    opt = torch.optim.AdamW(model.parameters(), lr=1e-3, weight_decay=0.0)
    engine = AxoNN_Inter_Layer_Engine(model, torch.nn.functional.cross_entropy,
                                      computation_dtype=torch.bfloat16 if use_cuda else torch.float32)
    loader = ax.create_dataloader(PrototypeDigits(args.samples), bs, mbs, shuffle=True)

    last = G_inter - 1 == ax.config.inter_layer_parallel_rank
    history = []
    for epoch in range(epochs):
        loader.sampler.set_epoch(epoch)
        for x, y in loader:
            opt.zero_grad(set_to_none=True)
            loss = engine.forward_backward_optimizer(x, y, opt)     # mean microbatch loss on the last stage
            history.append(float(loss))
    # the last stage of data-parallel replica 0 reports (the loss is 0 on the other stages)
    final = sum(history[-4:]) / 4
    ok = True
    if last and ax.config.data_parallel_rank == 0:
        print(json.dumps({"G_inter": G_inter, "G_data": G_data, "batch_size": bs, "micro_batch_size": mbs,
                          "steps": len(history), "first_loss": round(history[0], 4), "final_loss": round(final, 4)}),
              flush=True)
        ok = final < args.target_loss
    flag = torch.tensor([1 if ok else 0], device=device)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if int(flag) else 1)


if __name__ == "__main__":
    main()
