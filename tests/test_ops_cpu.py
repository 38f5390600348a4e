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
