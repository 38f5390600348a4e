"""Tensor-parallel Conv2d and Embedding against their torch.nn counterparts,
auto_parallelize, the Lightning-style strategy and the Transformers shim, on
CPU ranks (the reference's conv/embedding tests are disabled upstream)."""

import os

import pytest
import torch

from _dist import run_distributed


def _conv_emb(rank, world, grid):
    import torch.distributed as dist

    from axonn_b200 import axonn as ax
    from axonn_b200.intra_layer import Conv2d, Embedding, optimize_communication
    from axonn_b200.intra_layer.communication import _gather

    r, c, d = grid
    ax.init(1, world // (r * c * d), r, c, d)
    ch = ax.comm_handle
    inner, outer, depth = (ch.inner_intra_layer_parallel_group, ch.outer_intra_layer_parallel_group,
                           ch.depth_intra_layer_parallel_group)
    torch.manual_seed(0)
    # ---- conv: same input on every rank (the layer scatters it), output gathered by the layer
    seq = torch.nn.Conv2d(8, 16, 3, padding=1)
    par = Conv2d(8, 16, 3, padding=1)
    par.load_state_dict(seq.state_dict())
    X = torch.randn(4, 8, 6, 6)
    G = torch.randn(4, 16, 6, 6)
    xs = X.clone().requires_grad_(True)
    seq(xs).backward(G)
    xp = X.clone().requires_grad_(True)
    with optimize_communication(True, True, False, False):
        yp = par(xp)
        yp.backward(G)
    assert torch.allclose(yp, seq(X), atol=1e-5), (yp - seq(X)).abs().max()
    gw = _gather(par.weight.grad, 0, depth).reshape(par.local_weight_shape)
    gw = _gather(_gather(gw, 1, inner), 0, outer)
    assert torch.allclose(gw, seq.weight.grad, atol=1e-4), (gw - seq.weight.grad).abs().max()
    assert torch.allclose(xp.grad, xs.grad, atol=1e-4)
    # grid-independent form of the parameters (and of anything laid out like them) and back
    assert torch.equal(par.full_tensor("weight"), seq.weight) and torch.equal(par.full_tensor("bias"), seq.bias)
    assert torch.equal(par.full_tensor("weight", par.weight.grad), gw)
    assert torch.equal(par.shard_tensor("weight", seq.weight.detach()), par.weight)
    assert torch.equal(par.shard_tensor("bias", seq.bias.detach()), par.bias)

    # ---- embedding (hidden over the row group; needs c == 1 in easy mode)
    if c == 1:
        seq_e = torch.nn.Embedding(64, 16)
        par_e = Embedding(64, 16)
        par_e.load_state_dict(seq_e.state_dict())
        ids = torch.randint(0, 64, (3, 5))
        ye = par_e(ids)
        assert torch.allclose(ye, seq_e(ids))
        Ge = torch.randn(3, 5, 16)
        ye.backward(Ge)
        seq_e(ids).backward(Ge)
        ge = _gather(par_e.weight.grad, 0, depth).reshape(64, -1)
        ge = _gather(ge, 1, par_e.hidden_group)
        # the depth reduce-scatter sums the gradients of all depth ranks; here they all looked up the same ids
        assert torch.allclose(ge / d, seq_e.weight.grad, atol=1e-5)
        assert torch.equal(par_e.full_tensor("weight"), seq_e.weight)
        assert torch.equal(par_e.shard_tensor("weight", seq_e.weight.detach()), par_e.weight)
    return True


@pytest.mark.parametrize("grid", [(2, 1, 1), (1, 2, 1), (1, 1, 2)])
def test_conv_and_embedding_world2(grid):
    assert all(run_distributed(_conv_emb, 2, grid))


def _strategy(rank, world, folder):
    import torch.distributed as dist

    from axonn_b200 import axonn as ax
    from axonn_b200.intra_layer import Linear
    from axonn_b200.lightning import AxonnStrategy

    s = AxonnStrategy(G_intra_r=2, overlap_communication=True)
    s.setup_environment()
    assert ax.config.G_data == world // 2 and s.distributed_sampler_kwargs == {"num_replicas": world, "rank": rank}
    torch.manual_seed(0)
    with s.module_init_context():
        model = torch.nn.Sequential(torch.nn.Linear(16, 32), torch.nn.ReLU(), torch.nn.Linear(32, 16),
                                    torch.nn.Linear(16, 3))
    assert isinstance(model[0], Linear) and isinstance(model[2], Linear)
    assert type(model[3]) is torch.nn.Linear  # 3 outputs do not divide over 2 ranks
    model = s.setup_module(model)
    opt = torch.optim.SGD(model.parameters(), lr=0.1)
    torch.manual_seed(10 + rank)
    x, y = torch.randn(4, 16), torch.randn(4, 3)
    losses = []
    for it in range(3):
        opt.zero_grad()
        with s.no_backward_sync(model, enabled=False):
            loss = torch.nn.functional.mse_loss(model(x), y)
            s.backward(loss, model)
        s.clip_gradients_norm(model, opt, 1.0)
        opt.step()
        losses.append(float(loss))
    s.save_checkpoint(os.path.join(folder, "last.ckpt"), {"model": model, "optimizer": opt, "step": 3})
    dist.barrier()
    w_before = model[0].weight.detach().clone()
    with torch.no_grad():
        model[0].weight.zero_()
    rest = s.load_checkpoint(os.path.join(folder, "last.ckpt"), {"model": model, "optimizer": opt})
    assert torch.equal(model[0].weight, w_before) and rest == {"step": 3}
    return losses


def test_strategy_standalone(tmp_path):
    out = run_distributed(_strategy, 4, str(tmp_path))
    assert all(l[2] < l[0] for l in out)
    assert sorted(os.listdir(tmp_path)) == ["tp_row_0_col_0_depth_0", "tp_row_1_col_0_depth_0"]


def _hf(rank, world):
    transformers = pytest.importorskip("transformers")
    from axonn_b200 import axonn as ax
    from axonn_b200.intra_layer import Linear
    from axonn_b200.models.transformers import parallelize, parallelize_model

    ax.init(1, 1, G_intra_r=2)
    cfg = transformers.LlamaConfig(hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                                   num_attention_heads=4, num_key_value_heads=2, vocab_size=128,
                                   max_position_embeddings=64)
    cfg.architectures = ["LlamaForCausalLM"]
    torch.manual_seed(0)
    ref = transformers.LlamaForCausalLM(cfg).eval()
    ids = torch.randint(0, 128, (2, 16), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        want = ref(ids).logits
    # (a) convert the built model in place
    import copy
    m = copy.deepcopy(ref)
    n = parallelize_model(m)
    assert n == 2 * 7
    half = ids[rank:rank + 1]  # easy mode: every rank feeds its own batch shard
    with torch.no_grad():
        got = m(half).logits
    assert torch.allclose(got, want[rank:rank + 1], atol=2e-4), (got - want[rank:rank + 1]).abs().max()
    # (b) build inside the context and load the reference weights
    with parallelize(cfg, strict=True):
        m2 = transformers.LlamaForCausalLM(cfg).eval()
    assert isinstance(m2.model.layers[0].mlp.down_proj, Linear)
    attn = m2.model.layers[0].self_attn
    # row-parallel attention in expert mode: q/k/v hold half of the heads, o_proj reduces over the row group
    assert attn.q_proj.expert_mode and attn.q_proj.local_out_features == 32 and attn.o_proj.transpose
    m2.load_state_dict(ref.state_dict())
    with torch.no_grad():
        got2 = m2(ids).logits          # expert mode: the batch is replicated over the row group
    assert torch.allclose(got2, want, atol=2e-4), (got2 - want).abs().max()
    return True


def _hf_arch(rank, world, arch, grid):
    """OPT / Mistral / Mixtral built inside ``parallelize``: same logits as the sequential model."""
    transformers = pytest.importorskip("transformers")
    from axonn_b200 import axonn as ax
    from axonn_b200.intra_layer import Linear
    from axonn_b200.models.transformers import parallelize

    r, c = grid
    ax.init(1, 1, G_intra_r=r, G_intra_c=c)
    if arch == "opt":
        cfg = transformers.OPTConfig(hidden_size=64, ffn_dim=128, num_hidden_layers=2, num_attention_heads=4,
                                     vocab_size=128, max_position_embeddings=64, word_embed_proj_dim=64)
        cls, name = transformers.OPTForCausalLM, "OPTForCausalLM"
    elif arch == "mistral":
        cfg = transformers.MistralConfig(hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                                         num_attention_heads=4, num_key_value_heads=2, vocab_size=128,
                                         max_position_embeddings=64, sliding_window=None)
        cls, name = transformers.MistralForCausalLM, "MistralForCausalLM"
    else:
        cfg = transformers.MixtralConfig(hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                                         num_attention_heads=4, num_key_value_heads=2, vocab_size=128,
                                         max_position_embeddings=64, num_local_experts=4, num_experts_per_tok=2,
                                         sliding_window=None)
        cls, name = transformers.MixtralForCausalLM, "MixtralForCausalLM"
    cfg.architectures = [name]
    torch.manual_seed(0)
    ref = cls(cfg).eval()
    ids = torch.randint(0, 128, (2, 16), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        want = ref(ids).logits
    with parallelize(cfg, strict=True):
        m = cls(cfg).eval()
    n_tp = sum(isinstance(x, Linear) for x in m.modules())
    assert n_tp >= 2 * 4, n_tp
    m.load_state_dict(ref.state_dict())
    expert = c == 1
    feed = ids if expert else ids[rank:rank + 1]
    with torch.no_grad():
        got = m(feed).logits
    target = want if expert else want[rank:rank + 1]
    assert torch.allclose(got, target, atol=3e-4), (got - target).abs().max()
    return True


@pytest.mark.parametrize("arch,grid", [("opt", (2, 1)), ("mistral", (2, 1)), ("mixtral", (2, 1)), ("opt", (1, 2))])
def test_transformers_architecture_patches(arch, grid):
    pytest.importorskip("transformers")
    assert all(run_distributed(_hf_arch, 2, arch, grid, timeout=400))


def test_transformers_shim_llama():
    pytest.importorskip("transformers")
    assert all(run_distributed(_hf, 2, timeout=400))


def _prune_run(rank, world):
    import torch

    from axonn_b200 import axonn as ax
    from axonn_b200.intra_layer import Linear, prune_gradients_, register_pruning_hooks

    ax.init(G_inter=1, G_data=1, G_intra_r=1, G_intra_c=1, G_intra_d=2)
    torch.manual_seed(0)
    lin = Linear(32, 16, expert_mode=True)
    x = torch.randn(4, 32)
    lin(x).square().sum().backward()
    n = lin.weight.grad.numel()
    assert prune_gradients_(lin, 0.25) == 1
    kept = int((lin.weight.grad != 0).sum())
    assert abs(kept - round(0.25 * n)) <= 1, (kept, n)
    assert lin.bias is None or (lin.bias.grad != 0).any()   # biases stay dense
    lin.zero_grad()
    handles = register_pruning_hooks(lin, 0.5)
    lin(x).square().sum().backward()
    kept = int((lin.weight.grad != 0).sum())
    assert abs(kept - round(0.5 * n)) <= 1, (kept, n)
    for h in handles:
        h.remove()
    return kept


def test_gradient_pruning_explicit_and_hooks():
    run_distributed(_prune_run, 2)
