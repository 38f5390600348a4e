"""Plain-PyTorch baseline of the pipelined VGG-16 configuration (``bench.py --config vgg16 --impl reference``).

The reference's pipeline engine (``axonn/inter_layer.py``) imports ``mpi4py`` unconditionally and moves
activations with CUDA-aware MPI; neither exists in this image, so the engine itself cannot run.  This file
restates its algorithm with stock PyTorch only (nothing from ``axonn_b200`` is imported): the stage split by
forward FLOPs, the message-driven schedule in which the first stage keeps ``G_inter`` microbatches in flight
and every stage alternates forward and backward work as messages arrive (for equal-cost microbatches this is
the one-forward-one-backward order), ``torch.distributed`` NCCL ``isend``/``irecv`` for the activations and
activation gradients, cuDNN convolutions under bf16 autocast, a per-tensor NCCL all-reduce of the gradients
over the data-parallel group (what the reference's ``sync_gradients`` does) and SGD with momentum.
"""

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

_CFG = [64, 64, "M", 128, 128, "M", 256, 256, 256, "M", 512, 512, 512, "M", 512, 512, 512, "M"]


def _units(image, classes):
    units, c, hw, i = [], 3, image, 0
    while i < len(_CFG):
        v = _CFG[i]
        pool = i + 1 < len(_CFG) and _CFG[i + 1] == "M"
        layers = [nn.Conv2d(c, v, 3, padding=1), nn.ReLU(inplace=True)] + ([nn.MaxPool2d(2, 2)] if pool else [])
        flops = 2 * c * v * 9 * hw * hw
        if pool:
            hw //= 2
        units.append((nn.Sequential(*layers), (v, hw, hw), flops))
        c = v
        i += 2 if pool else 1
    feat = c * hw * hw
    units.append((nn.Sequential(nn.Flatten(), nn.Linear(feat, 4096), nn.ReLU(inplace=True)), (4096,), 2 * feat * 4096))
    units.append((nn.Sequential(nn.Linear(4096, 4096), nn.ReLU(inplace=True)), (4096,), 2 * 4096 * 4096))
    units.append((nn.Linear(4096, classes), (classes,), 2 * 4096 * classes))
    return units


def _partition(flops, stages):
    """Contiguous split minimising the largest part (small exhaustive search: 16 units, at most 4 stages)."""
    import itertools

    n, best = len(flops), None
    for cuts in itertools.combinations(range(1, n), stages - 1):
        b = (0,) + cuts + (n,)
        worst = max(sum(flops[b[k]:b[k + 1]]) for k in range(stages))
        if best is None or worst < best[0]:
            best = (worst, b)
    return best[1]


def build(device, rank, world, G_inter, G_data, image, classes, micro):
    """Return train_step(images, labels) -> loss (float; the last stage's value, 0 elsewhere)."""
    # rank layout of the reference: world_rank = data_rank * G_inter + inter_rank
    stage, replica = rank % G_inter, rank // G_inter
    torch.manual_seed(1234)
    units = _units(image, classes)
    b = _partition([u[2] for u in units], G_inter)
    body = nn.Sequential(*[units[i][0] for i in range(b[stage], b[stage + 1])]).to(device)
    in_shape = (3, image, image) if stage == 0 else units[b[stage] - 1][1]
    opt = torch.optim.SGD(body.parameters(), lr=0.01, momentum=0.9)
    first, last = stage == 0, stage == G_inter - 1
    prev_rank, next_rank = rank - 1, rank + 1
    dp_group = None
    for s in range(G_inter):   # every rank creates every group
        g = dist.new_group([r * G_inter + s for r in range(G_data)], backend="nccl")
        if s == stage:
            dp_group = g
    # one communicator per neighbour pair and direction: a communicator's transfers are FIFO, and a stage's
    # forward sends must not queue behind the backward sends of its neighbour (MPI tags in the reference)
    fw_group, bw_group = {}, {}
    for r in range(G_data):
        for s in range(G_inter - 1):
            a = r * G_inter + s
            gf = dist.new_group([a, a + 1], backend="nccl")
            gb = dist.new_group([a, a + 1], backend="nccl")
            if rank in (a, a + 1):
                fw_group[a], bw_group[a] = gf, gb

    def train_step(images, labels):
        n = images.shape[0] // micro
        opt.zero_grad(set_to_none=True)
        inputs, outputs, sends = {}, {}, []
        loss_sum = torch.zeros((), device=device)

        def forward(k):
            if first:
                x = images[k * micro:(k + 1) * micro]
            else:
                x = torch.empty((micro,) + tuple(in_shape), device=device, dtype=torch.bfloat16)
                dist.recv(x, src=prev_rank, group=fw_group[prev_rank])
                x.requires_grad_(True)
            with torch.autocast("cuda", dtype=torch.bfloat16):
                y = body(x)
            inputs[k], outputs[k] = x, y
            if not last:
                sends.append(dist.isend(y.detach().to(torch.bfloat16).contiguous(), dst=next_rank, group=fw_group[rank]))

        def backward(k):
            nonlocal loss_sum
            x, y = inputs.pop(k), outputs.pop(k)
            if last:
                loss = F.cross_entropy(y.float(), labels[k * micro:(k + 1) * micro]) / n
                loss_sum = loss_sum + loss.detach()
                loss.backward()
            else:
                g = torch.empty_like(y, dtype=torch.bfloat16)
                dist.recv(g, src=next_rank, group=bw_group[rank])
                y.backward(g.to(y.dtype))
            if not first:
                sends.append(dist.isend(x.grad.to(torch.bfloat16).contiguous(), dst=prev_rank, group=bw_group[prev_rank]))

        # warm-up forwards (stage s holds G_inter - s microbatches before its first backward), then one
        # forward / one backward, then the remaining backwards
        warm = min(G_inter - stage, n)
        for k in range(warm):
            forward(k)
        nf, nb = warm, 0
        while nb < n:
            backward(nb)
            nb += 1
            if nf < n:
                forward(nf)
                nf += 1
        for s in sends:
            s.wait()
        if G_data > 1:
            for p in body.parameters():
                if p.grad is not None:
                    dist.all_reduce(p.grad, group=dp_group)
                    p.grad.div_(G_data)
        opt.step()
        return float(loss_sum.item())

    return train_step
