"""Headline benchmark: GPT-1.3B training throughput (tokens/s, MFU) on N B200s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

N > 1 is launched by ``python -m torch.distributed.run --nproc-per-node N ...``
(RANK / LOCAL_RANK / WORLD_SIZE / MASTER_* from the environment).  Rank 0
prints one JSON line.  Configuration: GPT-style decoder 1.3B (24 layers,
d_model 2048, 16 heads, FFN 8192 GELU, LayerNorm, learned positions, vocab
50304, seq 2048), bf16 compute with fp32 master weights, AdamW, synthetic
uniform-random tokens, random-init weights; weak scaling with 8 sequences per
GPU (global batch 64 at 8 GPUs), each replica's batch in one microbatch (at most 32 sequences); the
tensor-parallel grid grows towards r=c=d=2: 1 -> (1,1,1), 2 -> d=2,
4 -> r=2,d=2, 8 -> r=c=d=2.

``value`` is device-timed (CUDA events, barrier + synchronize on both sides,
max over ranks) with the batch already resident on the GPU.  ``e2e`` times the
public call ``Trainer.train_step(host_tokens, host_targets)``, which copies the
step's batch from pinned host memory and reads the loss back every step.
"""

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

GRIDS = {1: (1, 1, 1), 2: (1, 1, 2), 4: (2, 1, 2), 8: (2, 2, 2)}  # (r, c, d)
SEQS_PER_GPU = 8
MICRO_BATCH = 32  # sequences per microbatch (upper bound; a replica's whole batch when it is smaller)


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="gpt1.3b", choices=["gpt1.3b", "tiny"])
    ap.add_argument("--no-e2e", action="store_true")
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


def main():
    args = parse()
    if args.impl == "reference":
        ref_dir = os.path.join(ROOT, "baseline", "_ref")
        if not os.path.isdir(os.path.join(ref_dir, "axonn", "intra_layer")):
            print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref does not hold the reference package"}))
            return
        sys.path.insert(0, ref_dir)
    import torch
    import torch.distributed as dist

    rank, world, local = init_distributed(args)
    dev = torch.device("cuda", local)
    r, c, d = GRIDS[world]
    from axonn_b200.models.gpt import GPTConfig

    cfg = GPTConfig.gpt_1p3b() if args.model == "gpt1.3b" else GPTConfig.tiny()
    replicas = d  # G_data = 1: the batch is split over the depth group only
    global_batch = SEQS_PER_GPU * world
    per_replica = global_batch // replicas
    micro = min(MICRO_BATCH, per_replica)

    launches = lambda: 0  # noqa: E731
    if args.impl == "ours":
        from axonn_b200 import axonn as ax
        from axonn_b200.models import GPT
        from axonn_b200.ops import _lib
        from axonn_b200.optim import FusedAdamW
        from axonn_b200.trainer import Trainer, replica_index

        ax.init(G_inter=1, G_data=1, G_intra_r=r, G_intra_c=c, G_intra_d=d)
        torch.manual_seed(1234)
        model = GPT(cfg, dtype=torch.bfloat16)
        opt = FusedAdamW(model.parameters(), lr=1e-4, weight_decay=0.01)
        trainer = Trainer(model, opt, micro_batch_size=micro)
        rep = replica_index()
        step_device = trainer.train_step_device
        step_e2e = trainer.train_step
        launches = lambda: _lib.launch_count  # noqa: E731
    else:
        import axonn as ref_axonn
        import axonn.intra_layer  # noqa: F401
        from axonn import axonn as rax

        sys.path.insert(0, os.path.join(ROOT, "baseline"))
        import reference_gpt

        rax.init(G_inter=1, G_data=1, G_intra_r=r, G_intra_c=c, G_intra_d=d)
        model, ref_step = reference_gpt.build(ref_axonn, cfg, dev)
        rep = rax.config.intra_layer_depth_parallel_rank

        def step_device(x, y):
            return ref_step(x, y, micro)

        def step_e2e(x, y):
            return float(ref_step(x.to(dev, non_blocking=True), y.to(dev, non_blocking=True), micro).item())

    # synthetic data: uniform random token ids, one distinct batch per step and replica
    g = torch.Generator().manual_seed(1000 + rep)
    n_batches = 4
    host = [torch.randint(0, cfg.vocab, (per_replica, cfg.seq_len + 1), generator=g) for _ in range(n_batches)]
    host_x = [h[:, :-1].contiguous().pin_memory() for h in host]
    host_y = [h[:, 1:].contiguous().pin_memory() for h in host]
    dev_x = [t.to(dev) for t in host_x]
    dev_y = [t.to(dev) for t in host_y]

    for i in range(args.warmup):
        step_device(dev_x[i % n_batches], dev_y[i % n_batches])
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()

    if args.profile:
        from torch.profiler import ProfilerActivity, profile

        with profile(activities=[ProfilerActivity.CUDA, ProfilerActivity.CPU]) as prof:
            step_device(dev_x[0], dev_y[0])
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
    l0 = launches()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        loss = step_device(dev_x[i % n_batches], dev_y[i % n_batches])
    e1.record()
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    n_launch = launches() - l0
    ms = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms_per_step = float(ms.item()) / args.steps
    final_loss = float(loss.item())

    if not args.no_e2e:
        step_e2e(host_x[0], host_y[0])
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for i in range(args.steps):
            step_e2e(host_x[i % n_batches], host_y[i % n_batches])
        torch.cuda.synchronize()
        t1 = time.perf_counter()
        dist.barrier()
        t = torch.tensor([(t1 - t0) * 1e3], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item()) / args.steps
    clocks = sampler.stop() if rank == 0 else None

    tokens_per_step = global_batch * cfg.seq_len
    value = tokens_per_step / (ms_per_step / 1e3)
    peak, peak_kind = measured_peak_tflops()
    flops_per_step = cfg.flops_per_token() * tokens_per_step
    mfu = flops_per_step / (ms_per_step / 1e3) / (world * peak * 1e12)
    if rank == 0:
        out = {
            "metric": "tokens/sec (GPT-1.3B training, device-timed, max over ranks)",
            "value": round(value, 1), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(ms_per_step, 3), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "impl": args.impl,
            "mfu": round(mfu, 4), "mfu_peak": f"{peak} TFLOP/s bf16 sustained, {peak_kind}",
            "loss": round(final_loss, 4),
            "config": {"model": "gpt-1.3b (24L, d2048, 16h, ffn8192, vocab50304)" if args.model == "gpt1.3b"
                       else "gpt-tiny", "global_batch": global_batch, "seq_len": cfg.seq_len,
                       "micro_batch": micro, "parallelism": f"r{r}c{c}d{d}", "optimizer": "AdamW",
                       "l2": "per-step working set (weights+activations, tens of GB) far exceeds the 126 MB L2"},
            "gpu_launches": n_launch,
            "clocks": clocks,
        }
        if not args.no_e2e:
            out["e2e"] = {"value": round(tokens_per_step / (e2e_ms / 1e3), 1), "unit": "tokens/s",
                          "ms_per_step": round(e2e_ms, 3),
                          "h2d_bytes_per_step": int(world * 2 * per_replica * cfg.seq_len * 8),
                          "d2h_bytes_per_step": 4 * world}
        print(json.dumps(out), flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
