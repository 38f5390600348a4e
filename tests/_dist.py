"""Spawn helper for multi-process tests (gloo on CPU, nccl on GPUs)."""

import os
import tempfile
import traceback

import torch
import torch.multiprocessing as mp


def _worker(rank, world, fn, init_file, backend, args, queue):
    try:
        import torch.distributed as dist

        os.environ["MASTER_ADDR"] = "127.0.0.1"
        if backend == "nccl":
            torch.cuda.set_device(rank)
        dist.init_process_group(backend, init_method=f"file://{init_file}", rank=rank, world_size=world)
        out = fn(rank, world, *args)
        dist.barrier()
        dist.destroy_process_group()
        queue.put((rank, None, out))
    except Exception:
        queue.put((rank, traceback.format_exc(), None))


def run_distributed(fn, world, *args, backend="gloo", timeout=240):
    """Run ``fn(rank, world, *args)`` on ``world`` processes; returns the list of
    per-rank results; raises with the first failing rank's traceback."""
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    with tempfile.TemporaryDirectory() as d:
        init_file = os.path.join(d, "rdzv")
        procs = [ctx.Process(target=_worker, args=(r, world, fn, init_file, backend, args, queue))
                 for r in range(world)]
        for p in procs:
            p.start()
        results, errors = {}, []
        try:
            for _ in range(world):
                rank, err, out = queue.get(timeout=timeout)
                if err:
                    errors.append((rank, err))
                    break
                results[rank] = out
        finally:
            for p in procs:
                p.join(timeout=5 if errors else 30)
                if p.is_alive():
                    p.kill()
        if errors:
            raise AssertionError(f"rank {errors[0][0]} failed:\n{errors[0][1]}")
    return [results[r] for r in range(world)]


_cache = {}


def run_cached(fn, world, *args, **kwargs):
    """``run_distributed`` whose result is remembered for the rest of the test session: single-process reference
    runs that several tests compare against are computed once."""
    key = (fn.__module__, fn.__name__, world, repr(args))
    if key not in _cache:
        _cache[key] = run_distributed(fn, world, *args, **kwargs)
    return _cache[key]
