"""The Fabric-facing subclass of ``AxonnStrategy`` (the branch taken when ``lightning`` is importable), run on CPU
ranks against a stand-in for the Lightning Fabric base classes (``tests/_fake_lightning.py``; Lightning itself is
not installed here).  The strategy brings up the process group through the cluster environment, builds the model
under its init context, trains through ``backward`` / ``clip_gradients_norm``, and writes and reads checkpoints
in the ``tp_row_R_col_C_depth_D`` layout; the result must equal plain single-process training."""

import os
import socket
import tempfile
import traceback

import pytest
import torch
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _train_plain(steps, X, Y):
    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(16, 32), torch.nn.Tanh(), torch.nn.Linear(32, 4))
    opt = torch.optim.SGD(model.parameters(), lr=0.1)
    losses = []
    for _ in range(steps):
        opt.zero_grad()
        loss = torch.nn.functional.cross_entropy(model(X), Y)
        loss.backward()
        torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
        opt.step()
        losses.append(float(loss.detach()))
    return losses


def _rank_main(rank, world, port, folder, queue):
    try:
        import _fake_lightning

        _fake_lightning.install()
        import torch.distributed as dist

        from axonn_b200 import axonn as ax
        from axonn_b200.lightning import axonn_strategy as mod

        assert mod.LIGHTNING_AVAILABLE and issubclass(mod.AxonnStrategy, _fake_lightning.ParallelStrategy)
        env = _fake_lightning.ClusterEnvironment(rank, world, port)
        s = mod.AxonnStrategy(parallel_devices=[torch.device("cpu")] * world, cluster_environment=env, G_intra_r=2,
                              overlap_communication=True, process_group_backend="gloo")
        s._configure_launcher()
        assert s.launcher.num_processes == world and s.num_nodes == 1 and s.process_group_backend == "gloo"
        s.setup_environment()
        assert dist.is_initialized() and dist.get_world_size() == world and s.G_data == world // 2
        assert ax.config.G_intra_r == 2 and s.root_device == torch.device("cpu")
        assert s.distributed_sampler_kwargs == {"num_replicas": world, "rank": rank}
        assert s.broadcast({"hello": rank}, src=0) == {"hello": 0}
        assert float(s.all_reduce(torch.tensor([float(rank)]), reduce_op="mean")) == (world - 1) / 2
        assert float(s.all_reduce(torch.tensor([1.0]), reduce_op="sum")) == world
        s.barrier()

        torch.manual_seed(0)
        with s.module_init_context():
            model = torch.nn.Sequential(torch.nn.Linear(16, 32), torch.nn.Tanh(), torch.nn.Linear(32, 4))
        from axonn_b200.intra_layer import Linear

        assert isinstance(model[0], Linear) and isinstance(model[2], Linear)
        torch.manual_seed(0)      # same start as the plain run (the parallel layer initialises its bias to zero)
        model.load_state_dict(torch.nn.Sequential(torch.nn.Linear(16, 32), torch.nn.Tanh(),
                                                  torch.nn.Linear(32, 4)).state_dict())
        s.module_to_device(model)
        model = s.setup_module(model)
        opt = torch.optim.SGD(model.parameters(), lr=0.1)
        g = torch.Generator().manual_seed(1)
        X, Y = torch.randn(8 * world, 16, generator=g), torch.randint(0, 4, (8 * world,), generator=g)
        x, y = X[rank * 8:(rank + 1) * 8], Y[rank * 8:(rank + 1) * 8]       # easy mode: one batch shard per rank
        losses = []
        for step in range(4):
            opt.zero_grad()
            loss = torch.nn.functional.cross_entropy(model(x), y)
            s.backward(loss, model)
            s.clip_gradients_norm(model, opt, 1.0)
            opt.step()
            losses.append(float(s.all_reduce(loss.detach().clone(), reduce_op="mean")))
            if step == 1:
                s.save_checkpoint(os.path.join(folder, "step2.ckpt"), {"model": model, "optimizer": opt, "step": 2})
                s.barrier()
        # the checkpoint lies under this rank's tensor-parallel prefix and restores the step-2 state
        path = s.sharded_path(os.path.join(folder, "step2.ckpt"))
        assert os.path.exists(path) and f"tp_row_{ax.config.intra_layer_row_parallel_rank}_col_0_depth_0" in path
        rest = s.load_checkpoint(os.path.join(folder, "step2.ckpt"), {"model": model, "optimizer": opt})
        assert rest == {"step": 2}
        again = []
        for _ in range(2):
            opt.zero_grad()
            loss = torch.nn.functional.cross_entropy(model(x), y)
            with s.no_backward_sync(model, enabled=False):
                s.backward(loss, model)
            s.clip_gradients_norm(model, opt, 1.0)
            opt.step()
            again.append(float(s.all_reduce(loss.detach().clone(), reduce_op="mean")))
        s.barrier()
        dist.destroy_process_group()
        queue.put((rank, None, (losses, again)))
    except Exception:
        queue.put((rank, traceback.format_exc(), None))


def test_fabric_subclass_trains_like_a_single_process():
    world = 4
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    port = _free_port()
    with tempfile.TemporaryDirectory() as folder:
        procs = [ctx.Process(target=_rank_main, args=(r, world, port, folder, queue)) for r in range(world)]
        for p in procs:
            p.start()
        results = {}
        try:
            for _ in range(world):
                rank, err, out = queue.get(timeout=300)
                assert err is None, f"rank {rank} failed:\n{err}"
                results[rank] = out
        finally:
            for p in procs:
                p.join(timeout=20)
                if p.is_alive():
                    p.kill()
    losses, again = results[0]
    g = torch.Generator().manual_seed(1)
    X, Y = torch.randn(8 * world, 16, generator=g), torch.randint(0, 4, (8 * world,), generator=g)
    ref = _train_plain(4, X, Y)
    assert losses == pytest.approx(ref, rel=1e-4)
    assert again == pytest.approx(ref[2:], rel=1e-4)        # resumed from the step-2 checkpoint
