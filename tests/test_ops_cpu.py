"""CPU fallbacks of the small ops and the host-side status helpers (no GPU, no process group)."""

import os

import pytest
import torch

from axonn_b200 import ops
from axonn_b200.ops import _lib


def test_column_sum_and_gelu_backward_colsum_cpu():
    torch.manual_seed(0)
    x = torch.randn(37, 24)
    dy = torch.randn(37, 24)
    assert torch.allclose(ops.column_sum(x), x.sum(0), atol=1e-5)
    dx, cs = ops.gelu_backward_colsum(dy, x)
    xr = x.clone().requires_grad_(True)
    torch.nn.functional.gelu(xr, approximate="tanh").backward(dy)
    assert torch.allclose(dx, xr.grad, atol=1e-5)
    assert torch.allclose(cs, xr.grad.sum(0), atol=1e-4)


def test_status_helpers_without_gpu():
    if torch.cuda.is_available():
        return
    assert _lib.device_status() == 0
    _lib.check_status()   # nothing to report
    e = _lib.AxonnCommTimeout(0x121)
    assert isinstance(e, _lib.KernelError) and e.status == 0x121 and "peer" in str(e)


def test_symm_canary_registry_is_empty_without_buffers():
    from axonn_b200.parallel import symm

    assert symm.verify_canaries() >= 0
    assert symm.debug_bounds_enabled() in (True, False)


def test_fused_adamw_state_dict_roundtrip_keeps_fp32_state_for_bf16_parameters():
    """Saving and reloading the optimizer in the middle of a run with bf16 parameters: master weights and
    moments stay fp32 and the next step is bit-identical to the uninterrupted run."""
    from axonn_b200.optim import FusedAdamW

    def make():
        torch.manual_seed(3)
        ps = [torch.nn.Parameter(torch.randn(33, 7).bfloat16()), torch.nn.Parameter(torch.randn(5).bfloat16())]
        return ps, FusedAdamW(ps, lr=1e-2, weight_decay=0.1)

    def grads(ps, seed):
        g = torch.Generator().manual_seed(seed)
        for p in ps:
            p.grad = torch.randn(p.shape, generator=g).bfloat16()

    ps_a, opt_a = make()
    ps_b, opt_b = make()
    for seed in (1, 2):
        grads(ps_a, seed); opt_a.step()
        grads(ps_b, seed); opt_b.step()
    # interrupted run: new optimizer object over the same parameter values, state loaded from a state dict
    ps_c = [torch.nn.Parameter(p.detach().clone()) for p in ps_b]
    opt_c = FusedAdamW(ps_c, lr=1e-2, weight_decay=0.1)
    sd = opt_b.state_dict()
    opt_c.load_state_dict(sd)
    for p in ps_c:
        st = opt_c.state[p]
        assert st["master"].dtype == torch.float32 and st["exp_avg"].dtype == torch.float32
        assert st["exp_avg_sq"].dtype == torch.float32
    grads(ps_a, 9); opt_a.step()
    grads(ps_c, 9); opt_c.step()
    for a, c in zip(ps_a, ps_c):
        assert torch.equal(a, c)
        assert torch.equal(opt_a.state[a]["master"], opt_c.state[c]["master"])


def test_fused_sgd_cpu_path_matches_torch_sgd():
    from axonn_b200.optim import FusedSGD

    torch.manual_seed(3)
    ours = [torch.nn.Parameter(torch.randn(7, 5)), torch.nn.Parameter(torch.randn(11))]
    ref = [torch.nn.Parameter(p.detach().clone()) for p in ours]
    a = FusedSGD(ours, lr=0.05, momentum=0.9, weight_decay=0.01)
    b = torch.optim.SGD(ref, lr=0.05, momentum=0.9, weight_decay=0.01)
    for _ in range(4):
        for p, q in zip(ours, ref):
            g = torch.randn_like(q)
            p.grad, q.grad = g.clone(), g.clone()
        a.step()
        b.step()
    for p, q in zip(ours, ref):
        assert torch.allclose(p, q, atol=1e-6)


def test_linear_batched_cpu_matches_per_expert_linear():
    from axonn_b200 import ops

    torch.manual_seed(4)
    x = torch.randn(3, 16, 8, requires_grad=True)
    w = torch.randn(3, 12, 8, requires_grad=True)
    seg = torch.tensor([[4, 8], [0, 8], [8, 8]], dtype=torch.int32)     # ignored by the CPU path: rows are not masked
    y = ops.linear_batched(x, w, seg, 8)
    ref = torch.stack([x[e] @ w[e].t() for e in range(3)])
    assert torch.allclose(y, ref, atol=1e-5)
    g = torch.randn_like(y)
    gx, gw = torch.autograd.grad(y, (x, w), g)
    rx, rw = torch.autograd.grad(ref, (x, w), g)
    assert torch.allclose(gx, rx, atol=1e-5) and torch.allclose(gw, rw, atol=1e-5)


def test_cpu_adam_state_dict_roundtrip_keeps_step_count_and_host_state():
    """Resuming from ``state_dict()`` continues exactly: the optimizer-wide step count (bias correction) and the
    flat host-side moments come back."""
    from axonn_b200.optim import CPUAdam

    torch.manual_seed(0)
    w0 = torch.randn(6, 5)
    grads = [torch.randn(6, 5) for _ in range(3)]

    def run(resume_after=None):
        p = torch.nn.Parameter(w0.clone())
        opt = CPUAdam([p], lr=1e-2, weight_decay=0.1)
        for i, g in enumerate(grads):
            if resume_after == i:
                sd = opt.state_dict()
                assert sd["steps"] == i
                q = torch.nn.Parameter(torch.zeros_like(p))
                opt = CPUAdam([q], lr=1.0)
                opt.load_state_dict(sd)
                assert opt.param_groups[0]["lr"] == 1e-2 and not opt.state[q]["exp_avg"].is_cuda
                p = q
            p.grad = g.clone()
            opt.step()
        return p.detach().clone()

    assert torch.equal(run(), run(resume_after=2))


def test_background_checkpoint_holds_the_values_of_the_call(tmp_path):
    """``save_async`` snapshots first and writes later: parameters changed right after the call do not leak into
    the file, a second call waits for the first, and a failing write surfaces in ``wait()``."""
    from axonn_b200 import checkpoint, config

    config.reset()
    model = torch.nn.Linear(64, 64)
    opt = torch.optim.SGD(model.parameters(), lr=0.1, momentum=0.9)
    model(torch.randn(4, 64)).sum().backward()
    opt.step()
    want = {k: v.clone() for k, v in model.state_dict().items()}
    state = {"model": model.state_dict(), "optimizer": opt.state_dict(), "step": 7}
    pending = checkpoint.save_async(state, str(tmp_path), "a")
    with torch.no_grad():
        for p in model.parameters():
            p.add_(1.0)                                   # the training loop goes on
    second = checkpoint.save_async({"model": model.state_dict(), "step": 8}, str(tmp_path), "b")
    assert pending.done()                                 # the second call waited for the first
    checkpoint.wait_for_pending_save()
    assert second.done() and second.wait() == checkpoint.checkpoint_path(str(tmp_path), "b")
    a = checkpoint.load(None, str(tmp_path), "a")
    b = checkpoint.load(None, str(tmp_path), "b")
    assert a["step"] == 7 and b["step"] == 8
    for k, v in want.items():
        assert torch.equal(a["model"][k], v) and torch.equal(b["model"][k], v + 1.0)
    assert torch.equal(a["optimizer"]["state"][0]["momentum_buffer"], opt.state_dict()["state"][0]["momentum_buffer"])
    with pytest.raises(ValueError):
        checkpoint.save_async(state, str(tmp_path), "a", overwrite=False)
    bad = checkpoint.save_async({"f": lambda: 0}, str(tmp_path), "c")     # not picklable: the writer thread fails
    with pytest.raises(Exception):
        bad.wait()
    assert not os.path.exists(checkpoint.checkpoint_path(str(tmp_path), "c"))


def test_upstream_import_names_resolve_after_the_alias_is_installed():
    """A script written against the upstream package's module names runs unchanged (child process: the alias
    changes ``sys.modules``)."""
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = r"""
import sys
sys.path.insert(0, %r)
import axonn_b200.compat
axonn_b200.compat.install_as_axonn()
axonn_b200.compat.install_as_axonn()          # idempotent
from axonn import axonn as ax
import axonn.config as config
from axonn.intra_layer import (Linear, Conv2d, Embedding, Drop, Gather, clip_grad_norm_, auto_parallelize,
                               optimize_communication, overlap_all_gathers_for_checkpointed_forward, no_grad_sync,
                               sync_gradients)
from axonn.intra_layer.communication import ForwardAllReduce, BackwardAllReduce, ForwardGather_BackwardReduceScatter
from axonn.intra_layer.fully_connected import extract_local_params_from_full_params
from axonn.inter_layer import AxoNN_Inter_Layer_Engine
from axonn.checkpoint import save, load, get_prefix_for_checkpoint
from axonn.lightning import AxonnStrategy
from axonn.models.transformers import parallelize
from axonn.timers import Timers
import axonn_b200
assert ax is axonn_b200.axonn and Linear is axonn_b200.intra_layer.Linear and config is axonn_b200.config
import torch, torch.distributed as dist, os
os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT="29731")
dist.init_process_group("gloo", rank=0, world_size=1)
ax.init(G_inter=1, G_data=1, G_intra_r=1, G_intra_c=1, G_intra_d=1)
with auto_parallelize():
    net = torch.nn.Linear(8, 8)
assert isinstance(net, Linear)
net(torch.randn(2, 8)).sum().backward()
sync_gradients(net)
print("alias ok")
""" % root
    r = subprocess.run([sys.executable, "-c", script], capture_output=True, text=True, timeout=300,
                       env=dict(os.environ, CUDA_VISIBLE_DEVICES=""))
    assert r.returncode == 0 and "alias ok" in r.stdout, r.stdout[-1500:] + r.stderr[-1500:]
