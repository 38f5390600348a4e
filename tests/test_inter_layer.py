"""Pipeline engine on CPU ranks: a ViT trained with G_inter=2 must follow the
same loss curve as with G_inter=1, data parallelism must compose with it, and
eval mode must not change the weights (pattern of the reference's
``axonn/tests/test_vit.py``, without the MNIST download)."""

import pytest
import torch

from _dist import run_cached, run_distributed


def _vit_run(rank, world, G_inter, G_data, steps, dtype_name):
    import torch.distributed as dist

    from axonn_b200 import axonn as ax
    from axonn_b200.inter_layer import AxoNN_Inter_Layer_Engine
    from axonn_b200.models import DistributedViT

    ax.init(G_inter=G_inter, G_data=G_data)
    dtype = getattr(torch, dtype_name)
    # build every stage with the same RNG stream so that all layouts share weights
    stages = []
    for s in range(G_inter):
        torch.manual_seed(100)
        full = [DistributedViT(image_size=16, patch_size=4, num_classes=10, dim=32, depth=4, heads=4,
                               mlp_dim=64, channels=1, G_inter=1, stage=0)]
        stages.append(full[0])
    full = stages[0]
    mine = DistributedViT(image_size=16, patch_size=4, num_classes=10, dim=32, depth=4, heads=4, mlp_dim=64,
                          channels=1)
    # copy the matching slice of the single-stage model
    sd = full.state_dict()
    per = 4 // G_inter
    stage = ax.config.inter_layer_parallel_rank
    new = {}
    for k, v in sd.items():
        if k.startswith("layers."):
            idx = int(k.split(".")[1])
            if stage * per <= idx < (stage + 1) * per:
                new["layers.%d.%s" % (idx - stage * per, k.split(".", 2)[2])] = v
        elif k in mine.state_dict():
            new[k] = v
    mine.load_state_dict(new)
    opt = torch.optim.SGD(mine.parameters(), lr=0.05)
    engine = AxoNN_Inter_Layer_Engine(mine, torch.nn.functional.cross_entropy, computation_dtype=dtype)
    ax.config.micro_batch_size = 4
    g = torch.Generator().manual_seed(3)
    X = torch.randn(16, 1, 16, 16, generator=g)
    Y = torch.randint(0, 10, (16,), generator=g)
    per_dp = 16 // G_data
    dp = ax.config.data_parallel_rank
    xb, yb = X[dp * per_dp:(dp + 1) * per_dp], Y[dp * per_dp:(dp + 1) * per_dp]
    losses = []
    for _ in range(steps):
        opt.zero_grad()
        losses.append(engine.forward_backward_optimizer(xb, yb, opt))
    ev = engine.forward_backward_optimizer(xb, yb, opt, eval_mode=True)
    # the loss lives on the last stage; average it over data-parallel replicas
    t = torch.tensor(losses + [ev], dtype=torch.float64)
    if ax.config.inter_layer_parallel_rank != G_inter - 1:
        t.zero_()
    dist.all_reduce(t)
    return (t / G_data).tolist()


def test_pipeline_matches_single_stage_fp32():
    ref = run_cached(_vit_run, 1, 1, 1, 4, "float32")[0]
    two = run_distributed(_vit_run, 2, 2, 1, 4, "float32")[0]
    assert two == pytest.approx(ref, rel=1e-5)
    assert ref[3] < ref[0]
    four = run_distributed(_vit_run, 4, 2, 2, 4, "float32")[0]
    assert four == pytest.approx(ref, rel=1e-4)


def test_fixed_order_schedule_matches_single_stage(monkeypatch):
    """The one-forward-one-backward order (what NCCL stages use when there are more than two) must give the same
    losses as a single stage, with two and with four stages."""
    ref = run_cached(_vit_run, 1, 1, 1, 4, "float32")[0]
    monkeypatch.setenv("AXONN_PIPELINE_SCHEDULE", "1f1b")
    four = run_distributed(_vit_run, 4, 4, 1, 4, "float32")[0]
    assert four == pytest.approx(ref, rel=1e-4)
    two = run_distributed(_vit_run, 4, 2, 2, 4, "float32")[0]
    assert two == pytest.approx(ref, rel=1e-4)


def test_pipeline_four_stages_bf16_trains():
    out = run_distributed(_vit_run, 4, 4, 1, 6, "bfloat16")[0]
    assert out[5] < out[0]


def test_vgg_partition_and_shapes():
    from axonn_b200.models.vgg import DistributedVGG16, _units, partition

    units = _units(224, 1000)
    assert len(units) == 16 and sum(1 for _ in units) == 13 + 3
    b = partition([u[2] for u in units], 4)
    assert b[0] == 0 and b[-1] == 16 and sorted(b) == b and len(b) == 5
    prev_out = None
    x = torch.randn(2, 3, 32, 32)
    for s in range(4):
        m = DistributedVGG16(image_size=32, num_classes=10, G_inter=4, stage=s)
        if prev_out is not None:
            assert m.get_input_shape()[1:] == prev_out
        x = m(x)
        assert list(x.shape[1:]) == m.get_output_shape()[1:]
        prev_out = m.get_output_shape()[1:]
    assert x.shape == (2, 10)


def _gpt_run(rank, world, G_inter, steps):
    import torch.distributed as dist
    import torch.nn.functional as F

    from axonn_b200 import axonn as ax
    from axonn_b200.inter_layer import AxoNN_Inter_Layer_Engine
    from axonn_b200.models import DistributedGPT, GPTConfig

    ax.init(G_inter=G_inter, G_data=1)
    cfg = GPTConfig(n_layers=4, hidden=32, n_heads=4, ffn=64, vocab=64, seq_len=16)
    torch.manual_seed(7)
    full = DistributedGPT(cfg, dtype=torch.float32, G_inter=1, stage=0)
    mine = DistributedGPT(cfg, dtype=torch.float32, ckp_coeff=2)
    per = cfg.n_layers // G_inter
    stage = ax.config.inter_layer_parallel_rank
    new = {}
    for k, v in full.state_dict().items():
        if k.startswith("blocks."):
            idx = int(k.split(".")[1])
            if stage * per <= idx < (stage + 1) * per:
                new["blocks.%d.%s" % (idx - stage * per, k.split(".", 2)[2])] = v
        elif k in mine.state_dict():
            new[k] = v
    mine.load_state_dict(new)
    assert mine.get_input_shape() == ([-1, 16] if stage == 0 else [-1, 16, 32])
    assert mine.get_output_shape() == ([-1, 16, 64] if stage == G_inter - 1 else [-1, 16, 32])
    opt = torch.optim.SGD(mine.parameters(), lr=0.1)
    loss_fn = lambda logits, y: F.cross_entropy(logits.reshape(-1, logits.shape[-1]), y.reshape(-1))  # noqa: E731
    engine = AxoNN_Inter_Layer_Engine(mine, loss_fn, computation_dtype=torch.float32)
    ax.config.micro_batch_size = 2
    g = torch.Generator().manual_seed(5)
    X = torch.randint(0, 64, (8, 16), generator=g)
    Y = torch.randint(0, 64, (8, 16), generator=g)
    losses = []
    for _ in range(steps):
        opt.zero_grad()
        losses.append(engine.forward_backward_optimizer(X, Y, opt))
    t = torch.tensor(losses, dtype=torch.float64)
    if stage != G_inter - 1:
        t.zero_()
    dist.all_reduce(t)
    return t.tolist()


def test_gpt_pipeline_stages_match_single_stage():
    ref = run_distributed(_gpt_run, 1, 1, 3)[0]
    two = run_distributed(_gpt_run, 2, 2, 3)[0]
    assert ref[-1] < ref[0]
    assert all(abs(a - b) < 1e-4 for a, b in zip(ref, two)), (ref, two)


def _fp16_scaling(rank, world):
    """fp16 through the pipeline with dynamic loss scaling: an overflowing batch skips the optimizer step on every
    stage and halves the scale; clean batches grow it back after the scaling window."""
    from axonn_b200 import axonn as ax
    from axonn_b200.inter_layer import AxoNN_Inter_Layer_Engine
    from axonn_b200.models import DistributedViT

    ax.init(G_inter=2, G_data=1)
    torch.manual_seed(20 + rank)
    model = DistributedViT(image_size=8, patch_size=4, num_classes=4, dim=16, depth=2, heads=2, mlp_dim=32, channels=1)
    opt = torch.optim.SGD(model.parameters(), lr=0.05)
    engine = AxoNN_Inter_Layer_Engine(model, torch.nn.functional.cross_entropy, computation_dtype=torch.float16)
    ax.config.micro_batch_size = 2
    g = torch.Generator().manual_seed(1)
    x, y = torch.randn(4, 1, 8, 8, generator=g), torch.randint(0, 4, (4,), generator=g)
    engine.scaler.scaling_window = 10 ** 9                    # first let the scale settle where fp16 holds the gradients
    for _ in range(12):
        start = engine.scaler.loss_scale
        opt.zero_grad()
        first = engine.forward_backward_optimizer(x, y, opt)
        if engine.scaler.loss_scale == start:
            break
    assert first == first and engine.scaler.loss_scale == start and start >= engine.scaler.min_scale
    engine.scaler.scaling_window, engine.scaler.no_overflow_iters = 2, 0
    before = [p.detach().clone() for p in model.parameters()]
    bad = x.clone()
    bad[0] = 6.0e4                                            # activations leave the fp16 range on the way
    opt.zero_grad()
    engine.forward_backward_optimizer(bad, y, opt)
    assert engine.scaler.loss_scale == start / 2              # every stage learned of the overflow ...
    assert all(torch.equal(a, b) for a, b in zip(before, model.parameters()))   # ... and skipped its update
    for _ in range(2):
        opt.zero_grad()
        loss = engine.forward_backward_optimizer(x, y, opt)
    assert engine.scaler.loss_scale == start and loss == loss
    assert any(not torch.equal(a, b) for a, b in zip(before, model.parameters()))
    return engine.scaler.loss_scale


def test_fp16_loss_scaling_skips_overflowing_steps_on_every_stage():
    a, b = run_distributed(_fp16_scaling, 2)
    assert a == b                                             # the stages agree on the scale


def _gpt_4d(rank, world, G_inter, G_data, r, c, d, steps):
    """Pipeline stages whose layers are tensor parallel, with data parallelism on top: all four dimensions."""
    import torch.distributed as dist

    from axonn_b200 import axonn as ax
    from axonn_b200 import ops
    from axonn_b200.inter_layer import AxoNN_Inter_Layer_Engine
    from axonn_b200.models import DistributedGPT, GPTConfig

    ax.init(G_inter=G_inter, G_data=G_data, G_intra_r=r, G_intra_c=c, G_intra_d=d)
    cfg = GPTConfig(n_layers=4, hidden=32, n_heads=4, ffn=64, vocab=64, seq_len=16)
    torch.manual_seed(7)
    full = DistributedGPT(cfg, dtype=torch.float32, G_inter=1, stage=0)        # same shards, all layers
    mine = DistributedGPT(cfg, dtype=torch.float32)
    per = cfg.n_layers // G_inter
    stage = ax.config.inter_layer_parallel_rank
    new = {}
    for k, v in full.state_dict().items():
        if k.startswith("blocks."):
            idx = int(k.split(".")[1])
            if stage * per <= idx < (stage + 1) * per:
                new["blocks.%d.%s" % (idx - stage * per, k.split(".", 2)[2])] = v
        elif k in mine.state_dict():
            new[k] = v
    mine.load_state_dict(new)
    group = mine.head.group if mine.last else None
    loss_fn = lambda logits, y: ops.cross_entropy(logits, y, group=group)  # noqa: E731  (vocabulary-parallel loss)
    engine = AxoNN_Inter_Layer_Engine(mine, loss_fn, computation_dtype=torch.float32)
    ax.config.micro_batch_size = 2
    g = torch.Generator().manual_seed(5)
    X = torch.randint(0, 64, (8, 16), generator=g)
    Y = torch.randint(0, 64, (8, 16), generator=g)
    replicas = G_data * d                                        # the batch is split over data and depth
    me = ax.config.G_intra_d * ax.config.data_parallel_rank + ax.config.intra_layer_depth_parallel_rank
    n = 8 // replicas
    xb, yb = X[me * n:(me + 1) * n], Y[me * n:(me + 1) * n]
    opt = torch.optim.SGD(mine.parameters(), lr=0.1)
    losses = []
    for _ in range(steps):
        opt.zero_grad()
        losses.append(engine.forward_backward_optimizer(xb, yb, opt))
    t = torch.tensor(losses, dtype=torch.float64)
    if stage != G_inter - 1:
        t.zero_()
    dist.all_reduce(t)                                           # last-stage ranks: tensor-parallel copies x replicas
    return (t / (r * c * d * G_data)).tolist()


_REF_4D = []


@pytest.mark.parametrize("layout", [(2, 1, 1, 2, 1), (2, 1, 1, 1, 2), (2, 2, 2, 1, 1)])
def test_gpt_pipeline_with_tensor_and_data_parallel_stages(layout):
    G_inter, G_data, r, c, d = layout
    if not _REF_4D:
        _REF_4D.append(run_distributed(_gpt_4d, 1, 1, 1, 1, 1, 1, 3)[0])
    ref = _REF_4D[0]
    world = G_inter * G_data * r * c * d
    got = run_distributed(_gpt_4d, world, G_inter, G_data, r, c, d, 3, timeout=400)[0]
    assert ref[-1] < ref[0]
    assert all(abs(a - b) < 2e-4 for a, b in zip(ref, got)), (layout, ref, got)
