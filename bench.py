"""Headline benchmark: training throughput on N B200s of one node.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config NAME]

N > 1 is launched by ``python -m torch.distributed.run --nproc-per-node N ...``
(RANK / LOCAL_RANK / WORLD_SIZE / MASTER_* from the environment).  Rank 0
prints one JSON line.

Configurations (``--config``; synthetic data of the named shape, random-init weights, bf16 compute):

  gpt1.3b (default)  GPT-style decoder 1.3B (24 layers, d_model 2048, 16 heads, FFN 8192 GELU, LayerNorm,
                     learned positions, vocab 50304, seq 2048), fp32 master weights, AdamW; weak scaling with 8
                     sequences per GPU (global batch 64 at 8 GPUs), each replica's batch in one microbatch (at
                     most 32 sequences); the tensor-parallel grid grows towards r=c=d=2:
                     1 -> (1,1,1), 2 -> d=2, 4 -> r=2,d=2, 8 -> r=c=d=2.
  llama8b            Llama-style 8B (32 layers, d_model 4096, 32/8 heads GQA, SwiGLU 14336, RMSNorm, RoPE,
                     vocab 128256, seq 4096), weights depth-sharded over all ranks (G_intra_d = N), 4 sequences
                     per GPU (global batch 32 at 8 GPUs) in microbatches of 2, AdamW, top-10 % gradient pruning.
  mixtral            Mixtral-style MoE (16 layers, d_model 4096, 8 SwiGLU experts of 14336, top-2), experts
                     partitioned over the data-parallel group (G_data = N), 2 sequences of 4096 per GPU (global
                     batch 16 at 8 GPUs), AdamW.
  vgg16              VGG-16 on 224x224 images through the pipeline engine, G_inter = min(4, N) x G_data = N /
                     G_inter, 32 images per GPU (global batch 256 at 8 GPUs) in microbatches of 32, SGD momentum.

``value`` is device-timed (CUDA events, barrier + synchronize on both sides,
max over ranks) with the batch already resident on the GPU.  ``e2e`` times the
public call (``Trainer.train_step(host_tokens, host_targets)`` or the engine's
``forward_backward_optimizer``), which copies the step's batch from pinned host
memory and reads the loss back every step.  ``exposed_comm_ms_per_step`` comes
from one extra, untimed, profiled step on rank 0: the time during which a
communication kernel runs and no compute kernel does, plus (ours) the time the
fused compute+collective kernels spent stalled on peers, measured inside them.
"""

import argparse
import json
import os
import subprocess
import sys
import threading
import time

# more hardware work queues than the default 8, set before the CUDA context exists: a pipeline stage keeps several
# blocking NCCL point-to-point kernels in flight beside its compute stream (both arms get the same setting)
os.environ.setdefault("CUDA_DEVICE_MAX_CONNECTIONS", "32")

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

GRIDS = {1: (1, 1, 1), 2: (1, 1, 2), 4: (2, 1, 2), 8: (2, 2, 2)}  # gpt1.3b: (r, c, d)
SEQS_PER_GPU = 8
MICRO_BATCH = 32  # gpt1.3b: sequences per microbatch (upper bound; a replica's whole batch when it is smaller)


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="gpt1.3b", choices=["gpt1.3b", "llama8b", "mixtral", "vgg16"])
    ap.add_argument("--model", default="full", choices=["full", "gpt1.3b", "tiny"],
                    help="'tiny' shrinks the model of the chosen configuration (smoke runs)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-exposed", action="store_true", help="skip the extra profiled step (exposed communication)")
    ap.add_argument("--ref-bf16-params", action="store_true",
                    help="reference arm, gpt1.3b: diagnostic line with the model cast to bf16 (no fp32 master "
                         "weights, no per-GEMM weight cast) to separate the recipe from the kernels")
    ap.add_argument("--profile", default=None, help="diagnostic: write a torch.profiler kernel table of one step "
                    "(rank 0) to this file and exit; no benchmark number is produced")
    return ap.parse_args()


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons of one GPU while a region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
                power.append(float(parts[2]))
            except ValueError:
                continue
            for nm, v in zip(names, parts[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


def init_distributed(args):
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", rank))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit(f"--gpus {args.gpus} needs a torch.distributed.run launch with {args.gpus} ranks")
        args.gpus = world
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29512")
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", local))
    return rank, world, local


def measured_peak_tflops():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["bf16_tflops_sustained"]), "measured"
    except Exception:
        return 1400.0, "fallback"


class Workload:
    """What a configuration hands to the timing loop."""

    def __init__(self, **kw):
        self.launches = lambda: 0
        self.check = lambda: None
        self.note = None
        self.__dict__.update(kw)


def _token_batches(torch, cfg, per_replica, rep, dev, n_batches=4):
    g = torch.Generator().manual_seed(1000 + rep)
    host = [torch.randint(0, cfg.vocab, (per_replica, cfg.seq_len + 1), generator=g) for _ in range(n_batches)]
    host_x = [h[:, :-1].contiguous().pin_memory() for h in host]
    host_y = [h[:, 1:].contiguous().pin_memory() for h in host]
    return host_x, host_y, [t.to(dev) for t in host_x], [t.to(dev) for t in host_y]


def _ours_lm(torch, model, opt, micro, prune=None):
    from axonn_b200.ops import _lib
    from axonn_b200.trainer import Trainer, replica_index

    trainer = Trainer(model, opt, micro_batch_size=micro, prune_keep_fraction=prune)
    return trainer, replica_index(), (lambda: _lib.launch_count), _lib.check_status


def build_gpt(args, torch, dist, rank, world, dev):
    r, c, d = GRIDS[world]
    from axonn_b200.models.gpt import GPTConfig

    cfg = GPTConfig.gpt_1p3b() if args.model != "tiny" else GPTConfig.tiny()
    replicas = d  # G_data = 1: the batch is split over the depth group only
    global_batch = SEQS_PER_GPU * world
    per_replica = global_batch // replicas
    micro = min(MICRO_BATCH, per_replica)
    w = Workload(cfg=cfg, units_per_step=global_batch * cfg.seq_len, unit="tokens/s",
                 flops_per_step=cfg.flops_per_token() * global_batch * cfg.seq_len,
                 metric="tokens/sec (GPT-1.3B training, device-timed, max over ranks)",
                 config={"model": "gpt-1.3b (24L, d2048, 16h, ffn8192, vocab50304)" if args.model != "tiny"
                         else "gpt-tiny", "global_batch": global_batch, "seq_len": cfg.seq_len,
                         "micro_batch": micro, "parallelism": f"r{r}c{c}d{d}", "optimizer": "AdamW",
                         "l2": "per-step working set (weights+activations, tens of GB) far exceeds the 126 MB L2"},
                 h2d=int(world * 2 * per_replica * cfg.seq_len * 8), d2h=4 * world)
    if args.impl == "ours":
        from axonn_b200 import axonn as ax
        from axonn_b200.models import GPT
        from axonn_b200.optim import FusedAdamW

        ax.init(G_inter=1, G_data=1, G_intra_r=r, G_intra_c=c, G_intra_d=d)
        torch.manual_seed(1234)
        model = GPT(cfg, dtype=torch.bfloat16)
        opt = FusedAdamW(model.parameters(), lr=1e-4, weight_decay=0.01)
        trainer, rep, w.launches, w.check = _ours_lm(torch, model, opt, micro)
        step_device, step_e2e = trainer.train_step_device, trainer.train_step
    else:
        import axonn as ref_axonn
        import axonn.intra_layer  # noqa: F401
        from axonn import axonn as rax

        sys.path.insert(0, os.path.join(ROOT, "baseline"))
        import reference_gpt

        rax.init(G_inter=1, G_data=1, G_intra_r=r, G_intra_c=c, G_intra_d=d)
        model, ref_step = reference_gpt.build(ref_axonn, cfg, dev, bf16_params=args.ref_bf16_params)
        rep = rax.config.intra_layer_depth_parallel_rank
        if args.ref_bf16_params:
            w.note = "diagnostic: reference model cast to bf16 (no fp32 master weights)"

        def step_device(x, y):
            return ref_step(x, y, micro)

        def step_e2e(x, y):
            return float(ref_step(x.to(dev, non_blocking=True), y.to(dev, non_blocking=True), micro).item())

    hx, hy, dx, dy = _token_batches(torch, cfg, per_replica, rep, dev)
    w.step_device = lambda i: step_device(dx[i % len(dx)], dy[i % len(dy)])
    w.step_e2e = lambda i: step_e2e(hx[i % len(hx)], hy[i % len(hy)])
    return w


def build_llama(args, torch, dist, rank, world, dev):
    from axonn_b200.models.llama import LlamaConfig

    cfg = LlamaConfig.llama_8b() if args.model != "tiny" else LlamaConfig.tiny()
    seqs_per_gpu, micro, keep = 4, 2, 0.1
    global_batch = seqs_per_gpu * world           # the batch is split over the depth group (= all ranks)
    w = Workload(cfg=cfg, units_per_step=global_batch * cfg.seq_len, unit="tokens/s",
                 flops_per_step=cfg.flops_per_token() * global_batch * cfg.seq_len,
                 metric="tokens/sec (Llama-8B training, depth-sharded weights, device-timed, max over ranks)",
                 config={"model": "llama-8b (32L, d4096, 32/8 heads, ffn14336, vocab128256)" if args.model != "tiny"
                         else "llama-tiny", "global_batch": global_batch, "seq_len": cfg.seq_len,
                         "micro_batch": micro, "parallelism": f"r1c1d{world}", "optimizer": "AdamW",
                         "gradient_pruning": "keep top 10 % |grad| per tensor",
                         "l2": "per-step working set (tens of GB) far exceeds the 126 MB L2"},
                 h2d=int(world * 2 * seqs_per_gpu * cfg.seq_len * 8), d2h=4 * world)
    if args.impl == "ours":
        from axonn_b200 import axonn as ax
        from axonn_b200.models import Llama
        from axonn_b200.optim import FusedAdamW

        ax.init(G_inter=1, G_data=1, G_intra_r=1, G_intra_c=1, G_intra_d=world)
        torch.manual_seed(1234)
        model = Llama(cfg, dtype=torch.bfloat16)
        opt = FusedAdamW(model.parameters(), lr=1e-4, weight_decay=0.01)
        trainer, rep, w.launches, w.check = _ours_lm(torch, model, opt, micro, prune=keep)
        step_device, step_e2e = trainer.train_step_device, trainer.train_step
    else:
        import axonn as ref_axonn
        import axonn.intra_layer  # noqa: F401
        from axonn import axonn as rax

        sys.path.insert(0, os.path.join(ROOT, "baseline"))
        import reference_llama

        rax.init(G_inter=1, G_data=1, G_intra_r=1, G_intra_c=1, G_intra_d=world)
        model, ref_step = reference_llama.build(ref_axonn, cfg, dev, prune_keep_fraction=keep)
        rep = rax.config.intra_layer_depth_parallel_rank
        w.note = "gradient pruning is not in the reference: plain torch.kthvalue threshold on its NCCL path"

        def step_device(x, y):
            return ref_step(x, y, micro)

        def step_e2e(x, y):
            return float(ref_step(x.to(dev, non_blocking=True), y.to(dev, non_blocking=True), micro).item())

    hx, hy, dx, dy = _token_batches(torch, cfg, seqs_per_gpu, rep, dev, n_batches=2)
    w.step_device = lambda i: step_device(dx[i % len(dx)], dy[i % len(dy)])
    w.step_e2e = lambda i: step_e2e(hx[i % len(hx)], hy[i % len(hy)])
    return w


def build_mixtral(args, torch, dist, rank, world, dev):
    from axonn_b200.models.mixtral import MixtralConfig

    cfg = MixtralConfig.mixtral_16l() if args.model != "tiny" else MixtralConfig.tiny()
    if args.model == "tiny":
        cfg.n_experts = max(4, world)
    seqs_per_gpu, micro = 2, 2
    global_batch = seqs_per_gpu * world
    w = Workload(cfg=cfg, units_per_step=global_batch * cfg.seq_len, unit="tokens/s",
                 flops_per_step=cfg.flops_per_token() * global_batch * cfg.seq_len,
                 metric="tokens/sec (Mixtral-style MoE training, expert parallel, device-timed, max over ranks)",
                 config={"model": "mixtral-16l (d4096, 32/8 heads, 8 experts x ffn14336, top-2, vocab32000)"
                         if args.model != "tiny" else "mixtral-tiny", "global_batch": global_batch,
                         "seq_len": cfg.seq_len, "micro_batch": micro, "parallelism": f"ep{world}",
                         "optimizer": "AdamW", "l2": "per-step working set (tens of GB) far exceeds the 126 MB L2"},
                 h2d=int(world * 2 * seqs_per_gpu * cfg.seq_len * 8), d2h=4 * world)
    if args.impl == "ours":
        from axonn_b200 import axonn as ax
        from axonn_b200.models import Mixtral
        from axonn_b200.optim import FusedAdamW

        ax.init(G_inter=1, G_data=world)
        torch.manual_seed(1234)
        model = Mixtral(cfg, dtype=torch.bfloat16)
        opt = FusedAdamW(model.parameters(), lr=1e-4, weight_decay=0.01)
        trainer, rep, w.launches, w.check = _ours_lm(torch, model, opt, micro)
        step_device, step_e2e = trainer.train_step_device, trainer.train_step
    else:
        sys.path.insert(0, os.path.join(ROOT, "baseline"))
        import reference_moe

        model, ref_step = reference_moe.build(cfg, dev, world, rank)
        rep = rank
        w.note = ("the reference has no expert parallelism: baseline = the same algorithm in plain PyTorch "
                  "(all_to_all_single dispatch/combine, per-expert cuBLAS GEMMs, NCCL gradient all-reduce)")

        def step_device(x, y):
            return ref_step(x, y, micro)

        def step_e2e(x, y):
            return float(ref_step(x.to(dev, non_blocking=True), y.to(dev, non_blocking=True), micro).item())

    hx, hy, dx, dy = _token_batches(torch, cfg, seqs_per_gpu, rep, dev, n_batches=2)
    w.step_device = lambda i: step_device(dx[i % len(dx)], dy[i % len(dy)])
    w.step_e2e = lambda i: step_e2e(hx[i % len(hx)], hy[i % len(hy)])
    return w


def build_vgg(args, torch, dist, rank, world, dev):
    tiny = args.model == "tiny"
    G_inter = 4 if world % 4 == 0 else (2 if world % 2 == 0 else 1)
    G_data = world // G_inter
    image, classes = (32, 10) if tiny else (224, 1000)
    per_gpu, micro = (4, 2) if tiny else (32, 32)
    global_batch = per_gpu * world
    per_replica = global_batch // G_data
    w = Workload(cfg=None, units_per_step=global_batch, unit="images/s",
                 flops_per_step=3 * 2 * 15.5e9 * global_batch,
                 metric="images/sec (VGG-16 training, inter-layer pipeline, device-timed, max over ranks)",
                 config={"model": "vgg-16 (13 conv 3x3 + 3 FC, no BatchNorm)" if not tiny else "vgg-tiny",
                         "global_batch": global_batch, "image": image, "micro_batch": micro,
                         "parallelism": f"G_inter{G_inter}xG_data{G_data}", "optimizer": "SGD momentum 0.9",
                         "l2": "activations of a microbatch (hundreds of MB) exceed the 126 MB L2"},
                 h2d=int(G_data * per_replica * (3 * image * image * 4 + 8)), d2h=4 * G_data)
    g = torch.Generator().manual_seed(7 + rank // G_inter)
    hx = torch.randn(per_replica, 3, image, image, generator=g).pin_memory()
    hy = torch.randint(0, classes, (per_replica,), generator=g).pin_memory()
    dx, dy = hx.to(dev), hy.to(dev)
    if args.impl == "ours":
        from axonn_b200 import axonn as ax
        from axonn_b200.inter_layer import AxoNN_Inter_Layer_Engine
        from axonn_b200.models import DistributedVGG16
        from axonn_b200.ops import _lib

        ax.init(G_inter=G_inter, G_data=G_data)
        torch.manual_seed(1234)
        model = DistributedVGG16(image_size=image, num_classes=classes).to(dev)
        from axonn_b200.optim import FusedSGD

        opt = FusedSGD(model.parameters(), lr=0.01, momentum=0.9)      # same update rule as the baseline's torch.optim.SGD
        engine = AxoNN_Inter_Layer_Engine(model, torch.nn.functional.cross_entropy, computation_dtype=torch.bfloat16)
        ax.config.micro_batch_size = micro
        w.launches, w.check = (lambda: _lib.launch_count), _lib.check_status

        def step(x, y):
            opt.zero_grad(set_to_none=True)
            return engine.forward_backward_optimizer(x, y, opt)

        w.step_device = lambda i: step(dx, dy)
        w.step_e2e = lambda i: step(hx, hy)
    else:
        sys.path.insert(0, os.path.join(ROOT, "baseline"))
        import reference_vgg

        ref_step = reference_vgg.build(dev, rank, world, G_inter, G_data, image, classes, micro)
        w.note = ("the reference's pipeline engine imports mpi4py (absent in this image): baseline = the same "
                  "message-driven schedule in plain PyTorch on NCCL p2p with cuDNN convolutions and an NCCL "
                  "gradient all-reduce")
        w.step_device = lambda i: ref_step(dx, dy)
        w.step_e2e = lambda i: ref_step(hx.to(dev, non_blocking=True), hy.to(dev, non_blocking=True))
    return w


BUILDERS = {"gpt1.3b": build_gpt, "llama8b": build_llama, "mixtral": build_mixtral, "vgg16": build_vgg}


def main():
    args = parse()
    dump_after = float(os.environ.get("AXONN_BENCH_DUMP_STACKS_S", "0") or 0)
    if dump_after > 0:
        # diagnostic for a run that stops making progress: every thread's Python stack on stderr after that many seconds
        import faulthandler

        faulthandler.dump_traceback_later(dump_after, exit=False)
    if args.impl == "reference" and args.config in ("gpt1.3b", "llama8b"):
        ref_dir = os.path.join(ROOT, "baseline", "_ref")
        if not os.path.isdir(os.path.join(ref_dir, "axonn", "intra_layer")):
            print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref does not hold the reference package"}))
            return
        sys.path.insert(0, ref_dir)
    import torch
    import torch.distributed as dist

    rank, world, local = init_distributed(args)
    dev = torch.device("cuda", local)
    w = BUILDERS[args.config](args, torch, dist, rank, world, dev)

    def as_float(loss):
        return float(loss.item()) if hasattr(loss, "item") else float(loss)

    for i in range(args.warmup):
        w.step_device(i)
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()

    if args.profile:
        from torch.profiler import ProfilerActivity, profile

        with profile(activities=[ProfilerActivity.CUDA, ProfilerActivity.CPU]) as prof:
            w.step_device(0)
            torch.cuda.synchronize()
        if rank == 0:
            with open(args.profile, "w") as f:
                f.write(prof.key_averages().table(sort_by="cuda_time_total", row_limit=45, max_name_column_width=90))
        dist.barrier()
        dist.destroy_process_group()
        return

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    l0 = w.launches()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        loss = w.step_device(i)
    e1.record()
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    n_launch = w.launches() - l0
    w.check()   # a device-side wait that ran out during the timed steps is an error, not a number
    ms = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms_per_step = float(ms.item()) / args.steps
    lt = torch.tensor([as_float(loss)], dtype=torch.float64, device=dev)
    dist.all_reduce(lt, op=dist.ReduceOp.MAX)   # pipelining: only the last stage holds the loss
    final_loss = float(lt.item())

    e2e_ms = None
    if not args.no_e2e:
        w.step_e2e(0)
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for i in range(args.steps):
            w.step_e2e(i)
        torch.cuda.synchronize()
        t1 = time.perf_counter()
        dist.barrier()
        t = torch.tensor([(t1 - t0) * 1e3], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item()) / args.steps
    clocks = sampler.stop() if rank == 0 else None

    exposed = None
    if not args.no_exposed:
        from axonn_b200.metrics import profile_exposed_comm

        dist.barrier()
        exposed = profile_exposed_comm(lambda: w.step_device(0), fused_stall=args.impl == "ours")
        torch.cuda.synchronize()
        dist.barrier()

    value = w.units_per_step / (ms_per_step / 1e3)
    peak, peak_kind = measured_peak_tflops()
    mfu = w.flops_per_step / (ms_per_step / 1e3) / (world * peak * 1e12)
    if rank == 0:
        out = {
            "metric": w.metric,
            "value": round(value, 1), "unit": w.unit, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(ms_per_step, 3), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "impl": args.impl,
            "mfu": round(mfu, 4), "mfu_peak": f"{peak} TFLOP/s bf16 sustained, {peak_kind}",
            "loss": round(final_loss, 4),
            "config": w.config,
            "gpu_launches": n_launch,
            "clocks": clocks,
        }
        if w.note:
            out["note"] = w.note
        if exposed is not None:
            out["exposed_comm_ms_per_step"] = round(exposed["exposed_comm_ms"] + exposed["fused_comm_stall_ms"], 3)
            out["exposed_comm"] = {
                "comm_kernels_not_covered_by_compute_ms": round(exposed["exposed_comm_ms"], 3),
                "stalled_on_peers_inside_fused_kernels_ms": round(exposed["fused_comm_stall_ms"], 3),
                "comm_kernel_ms": round(exposed["comm_kernel_ms"], 3),
                "compute_kernel_ms": round(exposed["compute_kernel_ms"], 3),
                "how": "one extra profiled step on rank 0: union of communication-kernel intervals minus union of "
                       "compute-kernel intervals; fused kernels count as compute and report their own stall time"}
        if e2e_ms is not None:
            out["e2e"] = {"value": round(w.units_per_step / (e2e_ms / 1e3), 1), "unit": w.unit,
                          "ms_per_step": round(e2e_ms, 3), "h2d_bytes_per_step": w.h2d, "d2h_bytes_per_step": w.d2h}
        print(json.dumps(out), flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
