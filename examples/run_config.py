"""Run one of the benchmark configurations end to end and print a JSON line.

    python -m torch.distributed.run --nproc-per-node 8 examples/run_config.py --config llama8b_depth
    python -m torch.distributed.run --nproc-per-node 8 examples/run_config.py --config mixtral_ep
    python -m torch.distributed.run --nproc-per-node 8 examples/run_config.py --config vgg16_pp

Configurations (synthetic data, random-init weights, bf16 compute, AdamW / SGD-momentum):

  llama8b_depth  Llama-style 8B, depth-sharded weights over all ranks (G_intra_d = world), global batch 32
                 sequences of 4096 tokens, top-10 % gradient pruning before the optimizer step
  mixtral_ep     Mixtral-style MoE (16 layers, 8 experts, top-2), experts partitioned over the data-parallel
                 group (G_data = world), global batch 16 sequences of 4096 tokens
  vgg16_pp       VGG-16 on 224x224 images, pipeline G_inter = 4 x G_data = world / 4, global batch 256 in
                 microbatches of 32, SGD momentum 0.9

``--scale tiny`` shrinks every model so that the same code path runs in seconds (used by the tests).
Timing: CUDA events around the timed steps, barrier + synchronize on both sides, max over ranks.
"""

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from axonn_b200 import axonn as ax  # noqa: E402
from axonn_b200.metrics import measured_peaks  # noqa: E402
from axonn_b200.optim import FusedAdamW  # noqa: E402
from axonn_b200.trainer import Trainer, num_replicas, replica_index  # noqa: E402


def timed(step, steps, warmup, device):
    for i in range(warmup):
        step(i)
    if device.type == "cuda":
        torch.cuda.synchronize()
    dist.barrier()
    if device.type == "cuda":
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
    import time

    t0 = time.perf_counter()
    out = None
    for i in range(steps):
        out = step(warmup + i)
    if device.type == "cuda":
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
    else:
        ms = (time.perf_counter() - t0) * 1e3
    dist.barrier()
    t = torch.tensor([ms], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item()) / steps, out


def run_lm(args, world, device, family):
    from axonn_b200.models import Llama, LlamaConfig, Mixtral, MixtralConfig

    tiny = args.scale == "tiny"
    if family == "llama":
        ax.init(G_inter=1, G_data=1, G_intra_r=1, G_intra_c=1, G_intra_d=world)
        cfg = LlamaConfig.tiny() if tiny else LlamaConfig.llama_8b()
        global_batch = 8 if tiny else 32
        model_cls, prune = Llama, 0.1
    else:
        ax.init(G_inter=1, G_data=world)
        cfg = MixtralConfig.tiny() if tiny else MixtralConfig.mixtral_16l()
        if tiny:
            cfg.n_experts = max(4, world)
        global_batch = 8 if tiny else 16
        model_cls, prune = Mixtral, None
    dtype = torch.bfloat16 if device.type == "cuda" else torch.float32
    torch.manual_seed(1234)
    model = model_cls(cfg, dtype=dtype)
    opt = FusedAdamW(model.parameters(), lr=1e-4, weight_decay=0.01)
    per = max(1, global_batch // num_replicas())
    trainer = Trainer(model, opt, micro_batch_size=min(per, args.micro_batch), prune_keep_fraction=prune, clip_grad=1.0)
    g = torch.Generator().manual_seed(100 + replica_index())
    data = [torch.randint(0, cfg.vocab, (per, cfg.seq_len + 1), generator=g) for _ in range(2)]
    xs = [d[:, :-1].contiguous().to(device) for d in data]
    ys = [d[:, 1:].contiguous().to(device) for d in data]
    ms, loss = timed(lambda i: trainer.train_step_device(xs[i % 2], ys[i % 2]), args.steps, args.warmup, device)
    tokens = per * num_replicas() * cfg.seq_len
    peak, _, kind = measured_peaks()
    return {"config": args.config, "metric": "tokens/s", "value": round(tokens / (ms / 1e3), 1),
            "ms_per_step": round(ms, 3), "mfu": round(cfg.flops_per_token() * tokens / (ms / 1e3) / (world * peak * 1e12), 4),
            "mfu_peak": f"{peak} TFLOP/s {kind}", "loss": round(float(loss), 4), "global_batch": per * num_replicas(),
            "seq_len": cfg.seq_len, "params": model.num_parameters()}


def run_vgg(args, world, device):
    from axonn_b200.inter_layer import AxoNN_Inter_Layer_Engine
    from axonn_b200.models import DistributedVGG16

    tiny = args.scale == "tiny"
    G_inter = 4 if world % 4 == 0 else (2 if world % 2 == 0 else 1)
    ax.init(G_inter=G_inter, G_data=world // G_inter)
    torch.manual_seed(1234)
    image, classes = (32, 10) if tiny else (224, 1000)
    model = DistributedVGG16(image_size=image, num_classes=classes).to(device)
    dtype = torch.bfloat16 if device.type == "cuda" else torch.float32
    opt = torch.optim.SGD(model.parameters(), lr=0.01, momentum=0.9)
    engine = AxoNN_Inter_Layer_Engine(model, torch.nn.functional.cross_entropy, computation_dtype=dtype)
    global_batch, micro = (16, 4) if tiny else (256, 32)
    per = global_batch // ax.config.G_data
    ax.config.micro_batch_size = micro
    g = torch.Generator().manual_seed(7 + ax.config.data_parallel_rank)
    x = torch.randn(per, 3, image, image, generator=g).to(device)
    y = torch.randint(0, classes, (per,), generator=g).to(device)

    def step(i):
        opt.zero_grad(set_to_none=True)
        return engine.forward_backward_optimizer(x, y, opt)

    ms, loss = timed(step, args.steps, args.warmup, device)
    t = torch.tensor([loss], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    peak, _, kind = measured_peaks()
    flops = DistributedVGG16(image_size=image, num_classes=classes, G_inter=1, stage=0).flops_per_image if tiny else \
        3 * 2 * 15.5e9
    return {"config": args.config, "metric": "images/s", "value": round(global_batch / (ms / 1e3), 1),
            "ms_per_step": round(ms, 3), "mfu": round(flops * global_batch / (ms / 1e3) / (world * peak * 1e12), 4),
            "loss": round(float(t.item()), 4), "global_batch": global_batch, "micro_batch": micro,
            "grid": f"G_inter={G_inter} x G_data={world // G_inter}"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", required=True, choices=["llama8b_depth", "mixtral_ep", "vgg16_pp"])
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--scale", default="full", choices=["full", "tiny"])
    ap.add_argument("--micro-batch", type=int, default=4)
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", rank))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29541")
    if torch.cuda.is_available():
        torch.cuda.set_device(local)
        device = torch.device("cuda", local)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    else:
        device = torch.device("cpu")
        dist.init_process_group("gloo", rank=rank, world_size=world)
    if args.config == "llama8b_depth":
        out = run_lm(args, world, device, "llama")
    elif args.config == "mixtral_ep":
        out = run_lm(args, world, device, "mixtral")
    else:
        out = run_vgg(args, world, device)
    out.update({"n_gpus": world, "steps": args.steps, "warmup": args.warmup, "data": "synthetic",
                "dtype": "bf16" if device.type == "cuda" else "fp32"})
    if rank == 0:
        print(json.dumps(out), flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
