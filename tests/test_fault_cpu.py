"""Failure detection without touching a GPU: a rank that stops participating
is reported by its peers' watchdogs, the pipeline engine's receive loop gives
up with PipelineTimeout instead of hanging, and training resumes from the
sharded checkpoint with the same loss."""

import os
import time

import pytest
import torch

from _dist import run_distributed


def _silent_rank(rank, world, tmp):
    from axonn_b200.parallel.watchdog import RankFailure, Watchdog

    wd = Watchdog(interval_s=0.1, timeout_s=1.0).start()
    time.sleep(0.5)
    wd.check()  # everybody alive
    if rank == 1:
        wd.stop()      # rank 1 goes silent (its process stays so that the test can finish cleanly)
        time.sleep(3.0)
        return "silent"
    time.sleep(2.5)
    try:
        wd.check()
    except RankFailure as e:
        wd.stop()
        return str(e)
    wd.stop()
    return "not detected"


def test_watchdog_reports_silent_rank(tmp_path):
    out = run_distributed(_silent_rank, 3, str(tmp_path))
    assert out[1] == "silent"
    assert "rank 1" in out[0] and "rank 1" in out[2]


def _pipeline_timeout(rank, world):
    from axonn_b200 import axonn as ax
    from axonn_b200.inter_layer import AxoNN_Inter_Layer_Engine, PipelineTimeout
    from axonn_b200.models import DistributedViT

    ax.init(G_inter=2, G_data=1)
    torch.manual_seed(0)
    model = DistributedViT(image_size=8, patch_size=4, num_classes=4, dim=16, depth=2, heads=2, mlp_dim=32, channels=1)
    eng = AxoNN_Inter_Layer_Engine(model, torch.nn.functional.cross_entropy, computation_dtype=torch.float32,
                                   timeout_s=1.5)
    ax.config.micro_batch_size = 2
    opt = torch.optim.SGD(model.parameters(), lr=0.1)
    if rank == 0:
        return "never joined the step"   # stage 0 does not send anything
    t0 = time.time()
    try:
        eng.forward_backward_optimizer(torch.zeros(4, 1, 8, 8), torch.zeros(4, dtype=torch.long), opt)
    except PipelineTimeout as e:
        return f"timeout after {time.time() - t0:.1f}s: {e}"
    return "no timeout"


def test_pipeline_receive_has_deadline():
    out = run_distributed(_pipeline_timeout, 2)
    assert out[1].startswith("timeout after") and "stage 1" in out[1]


def _ckpt_resume(rank, world, folder, phase):
    from axonn_b200 import axonn as ax
    from axonn_b200 import checkpoint
    from axonn_b200.models import GPT, GPTConfig
    from axonn_b200.optim import FusedAdamW
    from axonn_b200.trainer import Trainer

    r, c, d = (2, 1, 1)
    if phase.startswith("resume_grid_"):
        r, c, d = (int(v) for v in phase.split("_")[2:])
    ax.init(G_inter=1, G_data=world // (r * c * d), G_intra_r=r, G_intra_c=c, G_intra_d=d)
    torch.manual_seed(3)
    cfg = GPTConfig.tiny()
    model = GPT(cfg, dtype=torch.float32)
    opt = FusedAdamW(model.parameters(), lr=1e-3, weight_decay=0.0)
    tr = Trainer(model, opt)
    g = torch.Generator().manual_seed(9)
    data = torch.randint(0, cfg.vocab, (4, cfg.seq_len + 1), generator=g)
    x, y = data[:, :-1].contiguous(), data[:, 1:].contiguous()
    if phase == "train":
        losses = [tr.train_step(x, y) for _ in range(2)]
        checkpoint.save({"model": model.state_dict(), "optimizer": opt.state_dict()}, folder, "step2")
        written = checkpoint.save_consolidated(model, opt, folder, "step2", extra={"step": 2})
        assert (written is not None) == (rank == 0)
        losses += [tr.train_step(x, y) for _ in range(2)]
        return losses
    if phase.startswith("resume_grid_"):
        assert checkpoint.load_consolidated(model, opt, folder, "step2") == {"step": 2}
        return [tr.train_step(x, y) for _ in range(2)]
    state = checkpoint.load(None, folder, "step2")
    model.load_state_dict(state["model"])
    opt.load_state_dict(state["optimizer"])
    return [tr.train_step(x, y) for _ in range(2)]


def test_resume_from_sharded_checkpoint_reproduces_loss(tmp_path):
    folder = str(tmp_path / "ckpt")
    full = run_distributed(_ckpt_resume, 2, folder, "train")[0]
    assert sorted(os.listdir(folder)) == ["step2.full.pt", "tp_row_0_col_0_depth_0", "tp_row_1_col_0_depth_0"]
    resumed = run_distributed(_ckpt_resume, 2, folder, "resume")[0]
    assert resumed == pytest.approx(full[2:], rel=1e-5)
    # elastic restart: the grid-independent file written at the same step is loaded on other grids (depth instead
    # of row parallelism, a data-parallel pair, four ranks) and the loss curve continues; column parallelism and a
    # single process are covered by the tutorial test and the MoE test
    assert "step2.full.pt" in os.listdir(folder)
    for world, grid in ((2, "1_1_2"), (2, "1_1_1"), (4, "2_1_2")):
        other = run_distributed(_ckpt_resume, world, folder, "resume_grid_" + grid)[0]
        assert other == pytest.approx(full[2:], rel=2e-4), (world, grid)


def _pipeline_consolidated(rank, world, folder):
    """Two pipeline stages x two data-parallel replicas: one consolidated file per stage, written by replica 0."""
    import torch

    from axonn_b200 import axonn as ax
    from axonn_b200 import checkpoint
    from axonn_b200.models import DistributedViT

    ax.init(G_inter=2, G_data=2)
    torch.manual_seed(11 + ax.config.inter_layer_parallel_rank)
    model = DistributedViT(image_size=8, patch_size=4, num_classes=4, dim=16, depth=2, heads=2, mlp_dim=32, channels=1)
    opt = torch.optim.SGD(model.parameters(), lr=0.1, momentum=0.9)
    for p in model.parameters():
        p.grad = torch.ones_like(p)
    opt.step()
    path = checkpoint.save_consolidated(model, opt, folder, "pp", extra={"stage": ax.config.inter_layer_parallel_rank})
    assert (path is not None) == (ax.config.data_parallel_rank == 0)
    want = {k: v.clone() for k, v in model.state_dict().items()}
    with torch.no_grad():
        for p in model.parameters():
            p.zero_()
    opt2 = torch.optim.SGD(model.parameters(), lr=0.1, momentum=0.9)
    import torch.distributed as dist

    dist.barrier()
    extra = checkpoint.load_consolidated(model, opt2, folder, "pp")
    assert extra == {"stage": ax.config.inter_layer_parallel_rank}
    assert all(torch.equal(v, model.state_dict()[k]) for k, v in want.items())
    p0 = next(iter(model.parameters()))
    assert torch.equal(opt2.state[p0]["momentum_buffer"], torch.ones_like(p0))
    return sorted(os.listdir(folder))


def test_consolidated_checkpoint_has_one_file_per_pipeline_stage(tmp_path):
    out = run_distributed(_pipeline_consolidated, 4, str(tmp_path))
    assert all(files == ["pp.full.inter_0.pt", "pp.full.inter_1.pt"] for files in out)


class _Crash(RuntimeError):
    pass


def _fit(rank, world, folder, grid, steps, crash_at):
    from axonn_b200 import axonn as ax
    from axonn_b200.models import GPT, GPTConfig
    from axonn_b200.optim import FusedAdamW
    from axonn_b200.trainer import Trainer, num_replicas, replica_index

    r, c, d = grid
    ax.init(G_inter=1, G_data=world // (r * c * d), G_intra_r=r, G_intra_c=c, G_intra_d=d)
    torch.manual_seed(3)
    cfg = GPTConfig.tiny()
    model = GPT(cfg, dtype=torch.float32)
    tr = Trainer(model, FusedAdamW(model.parameters(), lr=1e-3, weight_decay=0.0))

    def batches(step):                      # a function of the step: global batch of 4, this replica's share
        g = torch.Generator().manual_seed(100 + step)
        data = torch.randint(0, cfg.vocab, (4, cfg.seq_len + 1), generator=g)
        per = 4 // num_replicas()
        mine = data[replica_index() * per:(replica_index() + 1) * per]
        return mine[:, :-1].contiguous(), mine[:, 1:].contiguous()

    def on_step(step, loss):
        if step == crash_at:
            raise _Crash(f"injected at step {step}")

    try:
        losses = tr.fit(batches, steps, checkpoint_folder=folder, checkpoint_every=2, on_step=on_step)
    except _Crash:
        return "crashed"
    import torch.distributed as dist

    out = {}
    for step, v in losses.items():          # replicas saw different samples: the global loss is their mean
        t = torch.tensor(v, dtype=torch.float64)
        dist.all_reduce(t)
        out[step] = float(t) / world
    return out


def test_fit_restarts_from_its_last_checkpoint_on_another_grid(tmp_path):
    """A run that dies after step 4 (checkpoints after steps 2 and 4) is started again on a different grid and
    finishes with the losses of a run that never stopped."""
    whole = run_distributed(_fit, 2, str(tmp_path / "a"), (2, 1, 1), 7, None)[0]
    assert sorted(whole) == list(range(7))
    folder = str(tmp_path / "b")
    assert run_distributed(_fit, 2, folder, (2, 1, 1), 7, 4) == ["crashed", "crashed"]
    assert open(os.path.join(folder, "latest")).read() == "step4"
    rest = run_distributed(_fit, 2, folder, (1, 1, 2), 7, None)[0]
    assert sorted(rest) == [4, 5, 6]
    for step in rest:
        assert rest[step] == pytest.approx(whole[step], rel=2e-4)


def _cpu_adam_moves(rank, world, folder, phase):
    """Host-resident optimizer state (CPUAdam keeps it flat, whatever the parameter's shape) through the
    grid-independent checkpoint: saved on a row-parallel grid, continued on a depth-parallel one."""
    from axonn_b200 import axonn as ax
    from axonn_b200 import checkpoint
    from axonn_b200.models import MLP
    from axonn_b200.optim import CPUAdam

    r, d = (2, 1) if phase != "resume" else (1, 2)
    ax.init(G_inter=1, G_data=1, G_intra_r=r, G_intra_d=d)
    torch.manual_seed(3)
    model = MLP(16, 32, 16, dtype=torch.float32)
    extra = torch.nn.Parameter(torch.ones(4, 4))              # a replicated 2-D parameter next to the sharded ones
    model.register_parameter("extra", extra)
    opt = CPUAdam(model.parameters(), lr=1e-2)
    g = torch.Generator().manual_seed(1)
    X = torch.randn(4, 16, generator=g)
    inner = ax.comm_handle.inner_intra_layer_parallel_group
    outer = ax.comm_handle.outer_intra_layer_parallel_group

    def step():
        from axonn_b200.intra_layer import sync_gradients
        from axonn_b200.intra_layer.communication import _drop, _gather

        opt.zero_grad()
        x = _drop(_drop(X, 0, ax.comm_handle.depth_intra_layer_parallel_group), 1, inner)
        y = model(x)
        loss = y.square().sum() * (model.extra.sum() / 16)
        loss.backward()
        sync_gradients(model, expert_mode=True)
        opt.step()
        total = _gather(loss.detach().reshape(1), 0, ax.comm_handle.depth_intra_layer_parallel_group).sum()
        return float(total)

    if phase == "whole":
        return [step() for _ in range(4)]
    if phase == "save":
        out = [step() for _ in range(2)]
        checkpoint.save_consolidated(model, opt, folder, "adam")
        return out
    checkpoint.load_consolidated(model, opt, folder, "adam")
    assert opt._steps == 2 and not opt.state[model.extra]["exp_avg"].is_cuda
    assert opt.state[model.extra]["exp_avg"].shape == (16,)   # flat host state of the 4 x 4 parameter
    return [step() for _ in range(2)]


def test_host_resident_optimizer_state_moves_between_grids(tmp_path):
    whole = run_distributed(_cpu_adam_moves, 2, str(tmp_path), "whole")[0]
    first = run_distributed(_cpu_adam_moves, 2, str(tmp_path), "save")[0]
    rest = run_distributed(_cpu_adam_moves, 2, str(tmp_path), "resume")[0]
    assert first + rest == pytest.approx(whole, rel=1e-4)
