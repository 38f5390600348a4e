"""Core runtime pieces on CPU ranks: the dataloader factory (which rank sees which samples, batch sizes with and
without pipelining) and the nested timers."""

import pytest
import torch

from _dist import run_distributed


class _Indices(torch.utils.data.Dataset):
    def __len__(self):
        return 64

    def __getitem__(self, i):
        return torch.tensor(i)


def _loader(rank, world, G_inter, G_data, r, c, d, global_batch, micro):
    from axonn_b200 import axonn as ax

    ax.init(G_inter=G_inter, G_data=G_data, G_intra_r=r, G_intra_c=c, G_intra_d=d)
    loader = ax.create_dataloader(_Indices(), global_batch, micro, shuffle=False)
    batches = [b.tolist() for b in loader]
    cfg = ax.config
    return dict(coords=(cfg.data_parallel_rank, cfg.inter_layer_parallel_rank, cfg.intra_layer_depth_parallel_rank,
                        cfg.intra_layer_row_parallel_rank, cfg.intra_layer_column_parallel_rank),
                batches=batches, per_gpu=cfg.batch_size_per_gpu, micro=cfg.micro_batch_size)


def test_dataloader_splits_samples_over_data_and_depth_only():
    """8 ranks as 2 (data) x 2 (depth) x 2 (row): four different sample streams, shared by the two row ranks of a
    (data, depth) pair; without pipelining the loader yields microbatches."""
    out = run_distributed(_loader, 8, 1, 2, 2, 1, 2, 16, 2)
    streams = {}
    for o in out:
        data, _, depth, row, _ = o["coords"]
        assert o["per_gpu"] == 4 and o["micro"] == 2 and all(len(b) == 2 for b in o["batches"])
        flat = [i for b in o["batches"] for i in b]
        streams.setdefault((data, depth), []).append(flat)
    assert len(streams) == 4
    seen = set()
    for (data, depth), copies in streams.items():
        assert len(copies) == 2 and copies[0] == copies[1]                  # the row ranks see the same samples
        replica = 2 * data + depth                                          # G_intra_d * data rank + depth rank
        assert copies[0] == list(range(replica, 64, 4))                     # DistributedSampler stride = replicas
        assert not seen & set(copies[0])
        seen |= set(copies[0])
    assert seen == set(range(64))


def test_dataloader_yields_whole_replica_batches_when_pipelining():
    out = run_distributed(_loader, 4, 2, 2, 1, 1, 1, 16, 4)
    for o in out:
        data, stage = o["coords"][0], o["coords"][1]
        assert o["per_gpu"] == 8 and all(len(b) == 8 for b in o["batches"])  # the engine cuts microbatches itself
        assert [i for b in o["batches"] for i in b] == list(range(data, 64, 2))
    assert out[0]["batches"] == out[1]["batches"]                            # both stages of a pipeline: same data


def _bad_batch(rank, world):
    from axonn_b200 import axonn as ax

    ax.init(G_inter=1, G_data=2)
    try:
        ax.create_dataloader(_Indices(), 10, 4)
    except ValueError as e:
        return str(e)
    return "accepted"


def test_dataloader_rejects_indivisible_batch():
    assert all("divisible" in m for m in run_distributed(_bad_batch, 2))


def test_nested_timers_key_regions_by_their_parents():
    import time

    from axonn_b200.timers import Timers

    t = Timers(use_cuda=False)
    for _ in range(3):
        t.start("step")
        t.start("comm")
        time.sleep(0.002)
        t.stop("comm")
        t.start("compute")
        t.start("comm")                     # the same inner key under another parent is another series
        t.stop("comm")
        t.stop("compute")
        t.stop("step")
    with pytest.raises(AssertionError):
        t.start("a")
        t.stop("b")
    t.stack.clear()
    t.open.clear()
    total, counts = t.get_times()
    assert counts == {("step",): 3, ("step", "comm"): 3, ("step", "compute"): 3, ("step", "compute", "comm"): 3}
    assert total[("step",)] >= total[("step", "comm")] >= 6.0 - 1e-6
    assert t.get_times() == ({}, {})         # reading resets
    off = Timers(enabled=False)
    off.start("x")
    off.stop("y")                            # disabled timers accept anything
    assert off.get_times() == ({}, {})


def test_exposed_communication_interval_arithmetic_matches_a_brute_force_timeline():
    """Union / subtraction of kernel intervals against a per-tick timeline, on random integer intervals."""
    import random

    from axonn_b200.metrics import exposed_comm_from_intervals

    rng = random.Random(7)
    for _ in range(200):
        kernels = []
        for _ in range(rng.randint(0, 12)):
            s = rng.randint(0, 60)
            e = s + rng.randint(0, 15)                       # empty intervals occur and must not count
            kernels.append((rng.choice(["ncclDevKernel_AllReduce", "gemm_pair_kernel", "axb::a2a_v_rows",
                                        "fa_fwd_pingpong_kernel"]), s, e))
        comm = [False] * 80
        comp = [False] * 80
        for name, s, e in kernels:
            line = comm if ("nccl" in name.lower() or "a2a_v" in name) else comp
            for t in range(s, e):
                line[t] = True
        want = (sum(c and not p for c, p in zip(comm, comp)), sum(comm), sum(comp))
        assert exposed_comm_from_intervals(kernels) == want, kernels


def test_step_meter_reports_throughput_and_writes_jsonl(tmp_path):
    import json
    import time

    from axonn_b200.metrics import StepMeter

    log = tmp_path / "steps.jsonl"
    meter = StepMeter(flops_per_token=1e9, world_size=1, log_path=str(log))
    meter.use_cuda = False                                    # host clock, whatever the machine has
    for _ in range(3):
        with meter.step(1000):
            time.sleep(0.01)
    out = meter.summary()
    assert out["steps"] == 3 and 10.0 <= out["ms_per_step"] < 200.0
    assert out["tokens_per_s"] == pytest.approx(3000 / (3 * out["ms_per_step"] / 1e3))
    assert out["mfu"] == pytest.approx(1e9 * out["tokens_per_s"] / (out["mfu_peak_tflops"] * 1e12))
    assert json.loads(log.read_text().splitlines()[-1])["steps"] == 3
    assert meter.summary()["steps"] == 0                      # reset after reading
