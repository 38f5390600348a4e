"""The bounds-checking build of the kernel library (``-DAXB_DEBUG_BOUNDS``): every computed offset into an inbox,
a flag array or an output tensor is verified before the store.  With correct index arithmetic the checks stay
silent - status word 0 - and the results equal those of the normal build.  Skipped unless the debug library
has been built (``python axonn_b200/utils/build.py --debug-bounds``)."""

import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DEBUG_LIB = os.path.join(ROOT, "axonn_b200", "lib", "libaxonn_b200_debug.so")

_CHILD = r"""
import sys, torch
sys.path.insert(0, %r)
from axonn_b200.ops import _lib
from axonn_b200.parallel import fused
assert _lib.LIB_PATH.endswith("libaxonn_b200_debug.so"), _lib.LIB_PATH
torch.manual_seed(0)
for (M, N, K) in [(4096, 4096, 512), (1000, 520, 264), (384, 136, 64)]:
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    ref = 2.0 * (a.float() @ b.float().t())
    for _ in range(2):
        one = fused.gemm_all_reduce_loopback(a, b)
        two, peer = fused.gemm_all_reduce_loopback(a, b, two_shot=True)
    torch.cuda.synchronize()
    st = _lib.device_status()
    assert st == 0, hex(st)
    assert (one.float() - ref).abs().max() <= 2e-2 * ref.abs().max()
    rows = torch.arange(M, device="cuda")
    owned = ((rows // 32) %% 2) == 0
    assert (two.float()[owned] - ref[owned]).abs().max() <= 2e-2 * ref.abs().max()
print("debug-bounds ok")
"""


def test_bounds_checked_kernels_stay_silent_on_correct_indices():
    if not os.path.exists(DEBUG_LIB):
        pytest.skip("debug library not built (python axonn_b200/utils/build.py --debug-bounds)")
    env = dict(os.environ, AXONN_DEBUG_BOUNDS="1")
    r = subprocess.run([sys.executable, "-c", _CHILD % ROOT], env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "debug-bounds ok" in r.stdout, r.stdout + r.stderr
