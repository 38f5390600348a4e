"""VGG-16 (13 conv 3x3 + 3 FC, no BatchNorm) split into pipeline stages.

``DistributedVGG16`` assigns consecutive units (conv+ReLU[+pool], then the
classifier layers) to ``G_inter`` stages with roughly equal forward FLOPs and
implements the pipeline engine's stage contract.  Workload of the reference's
``examples/test_vgg16.py`` (torchvision VGG-16 on 3x224x224 inputs, 1000
classes) without depending on torchvision.
"""

import torch.nn as nn

from .. import axonn as ax

_CFG = [64, 64, "M", 128, 128, "M", 256, 256, 256, "M", 512, 512, 512, "M", 512, 512, 512, "M"]


def _units(image_size, num_classes, channels=3):
    """List of (module factory, output shape (C,H,W) or (F,), flops)."""
    units, c, hw = [], channels, image_size
    i = 0
    while i < len(_CFG):
        v = _CFG[i]
        pool = i + 1 < len(_CFG) and _CFG[i + 1] == "M"
        cin, cout, res = c, v, hw

        def make(cin=cin, cout=cout, pool=pool):
            layers = [nn.Conv2d(cin, cout, 3, padding=1), nn.ReLU(inplace=True)]
            if pool:
                layers.append(nn.MaxPool2d(2, 2))
            return nn.Sequential(*layers)

        flops = 2 * cin * cout * 9 * res * res
        if pool:
            hw //= 2
        units.append((make, (cout, hw, hw), flops))
        c = cout
        i += 2 if pool else 1
    feat = c * hw * hw
    units.append((lambda f=feat: nn.Sequential(nn.Flatten(), nn.Linear(f, 4096), nn.ReLU(inplace=True)), (4096,),
                  2 * feat * 4096))
    units.append((lambda: nn.Sequential(nn.Linear(4096, 4096), nn.ReLU(inplace=True)), (4096,), 2 * 4096 * 4096))
    units.append((lambda: nn.Linear(4096, num_classes), (num_classes,), 2 * 4096 * num_classes))
    return units


def partition(flops, stages):
    """Contiguous split of ``flops`` into ``stages`` parts minimising the largest part."""
    n = len(flops)
    best = None

    def rec(start, k, cuts, worst):
        nonlocal best
        if k == 1:
            w = max(worst, sum(flops[start:]))
            if best is None or w < best[0]:
                best = (w, cuts + [n])
            return
        acc = 0
        for end in range(start + 1, n - k + 2):
            acc += flops[end - 1]
            if best is not None and acc >= best[0]:
                break
            rec(end, k - 1, cuts + [end], max(worst, acc))

    rec(0, stages, [], 0)
    return [0] + best[1]


class DistributedVGG16(nn.Module):
    """One pipeline stage of VGG-16: the network's units (convolution blocks, classifier layers) are dealt to the
    ``G_inter`` stages so that their forward FLOPs balance; same stage contract as ``DistributedViT``."""

    def __init__(self, image_size=224, num_classes=1000, channels=3, G_inter=None, stage=None):
        super().__init__()
        G_inter = ax.config.G_inter if G_inter is None else G_inter
        stage = ax.config.inter_layer_parallel_rank if stage is None else stage
        units = _units(image_size, num_classes, channels)
        bounds = partition([u[2] for u in units], G_inter)
        lo, hi = bounds[stage], bounds[stage + 1]
        self.stage, self.G_inter = stage, G_inter
        self.body = nn.Sequential(*[units[i][0]() for i in range(lo, hi)])
        self.in_shape = [channels, image_size, image_size] if lo == 0 else list(units[lo - 1][1])
        self.out_shape = list(units[hi - 1][1])
        self.flops_per_image = 3 * sum(u[2] for u in units)  # fwd + bwd

    def get_input_shape(self):
        return [-1] + self.in_shape

    def get_output_shape(self):
        return [-1] + self.out_shape

    def forward(self, x):
        return self.body(x)
