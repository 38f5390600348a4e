"""CPU fallbacks of the small ops and the host-side status helpers (no GPU, no process group)."""

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
