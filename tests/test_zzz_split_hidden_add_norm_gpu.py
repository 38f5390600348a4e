"""The fused residual-add + norm with the hidden dimension split over two ranks, emulated on one GPU.

With column tensor parallelism every rank holds a slice of the hidden dimension, so the norm runs as two launches
around an all-reduce of the per-row sums: forward mode 1 (h = x + delta written, partial sums) -> sum over ranks ->
mode 3 (finish the statistics in place, apply them); backward mode 1 (partial sums of g*dy and g*dy*xhat) -> sum
over ranks -> mode 2 (input gradient plus the gradient of the residual path, parameter gradients).  Here the two
slices are processed one after the other and the all-reduce is a plain addition; the result must equal the norm of
the whole row evaluated in fp32."""

import ctypes

import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _close(a, b, rel, abs_=1e-3):
    a, b = a.float(), b.float()
    err = (a - b).abs().max().item()
    assert err <= rel * b.abs().max().item() + abs_, f"max err {err} vs scale {b.abs().max().item()}"


@pytest.mark.parametrize("rms", [False, True])
def test_add_norm_split_hidden_forward_and_backward(rms):
    from axonn_b200.ops import _lib

    torch.manual_seed(6)
    rows, H, n = 261, 2048, 2
    Hl = H // n
    L = _lib.lib()
    x = torch.randn(rows, H, device=DEV).bfloat16()
    dl = torch.randn(rows, H, device=DEV).bfloat16()
    g = (1 + 0.1 * torch.randn(H, device=DEV)).bfloat16()
    b = (0.1 * torch.randn(H, device=DEV)).bfloat16()
    dy = torch.randn(rows, H, device=DEV).bfloat16()
    dres = torch.randn(rows, H, device=DEV).bfloat16()

    def sl(t, i):
        return t[..., i * Hl:(i + 1) * Hl].contiguous()

    xs, ds, gs, bs = ([sl(t, i) for i in range(n)] for t in (x, dl, g, b))
    dys, drs = ([sl(t, i) for i in range(n)] for t in (dy, dres))
    hs = [torch.empty_like(t) for t in xs]
    ys = [torch.empty_like(t) for t in xs]
    stats = [torch.empty(rows, 2, dtype=torch.float32, device=DEV) for _ in range(n)]

    def fwd(i, mode):
        src, delta, hout = (xs[i], ds[i], hs[i]) if mode == 1 else (hs[i], None, None)
        st = L.axb_add_norm_fwd(_lib.ptr(src), _lib.ptr(delta), _lib.ptr(hout), _lib.ptr(gs[i]),
                                _lib.ptr(None if rms else bs[i]), _lib.ptr(ys[i]), _lib.ptr(stats[i]),
                                ctypes.c_int(rows), ctypes.c_int(Hl), ctypes.c_int(H), ctypes.c_float(1e-5),
                                ctypes.c_int(1 if rms else 0), ctypes.c_int(mode), ctypes.c_int(0), ctypes.c_int(0),
                                _lib.stream_ptr())
        _lib.check(st, "axb_add_norm_fwd")

    for i in range(n):
        fwd(i, 1)
    total = stats[0] + stats[1]
    for i in range(n):
        stats[i].copy_(total)
        fwd(i, 3)
    h = torch.cat(hs, 1)
    y = torch.cat(ys, 1)
    assert torch.equal(h, x + dl)                                   # the same rounding as a separate add

    hr = h.float().requires_grad_(True)
    gr, br = g.float().requires_grad_(True), b.float().requires_grad_(True)
    if rms:
        yr = hr * torch.rsqrt(hr.pow(2).mean(-1, keepdim=True) + 1e-5) * gr
    else:
        yr = F.layer_norm(hr, (H,), gr, br, 1e-5)
    _close(y, yr, 1e-2)
    assert torch.equal(stats[0], stats[1])                          # (mean, rstd) of the whole row on both slices

    # ---- backward
    grid = int(L.axb_norm_grid(ctypes.c_int(0), ctypes.c_int(rows)))
    dxs = [torch.empty_like(t) for t in xs]
    sums = [torch.empty(rows, 2, dtype=torch.float32, device=DEV) for _ in range(n)]
    parts = [torch.empty(2, grid, Hl, dtype=torch.float32, device=DEV) for _ in range(n)]
    dgbs = [torch.empty(2, Hl, dtype=torch.bfloat16, device=DEV) for _ in range(n)]

    def bwd(i, mode):
        st = L.axb_add_norm_bwd(_lib.ptr(dys[i]), _lib.ptr(drs[i]), _lib.ptr(hs[i]), _lib.ptr(gs[i]),
                                _lib.ptr(stats[i]), _lib.ptr(dxs[i]), _lib.ptr(sums[i]), _lib.ptr(parts[i][0]),
                                _lib.ptr(parts[i][1]), _lib.ptr(dgbs[i][0]), _lib.ptr(dgbs[i][1]), ctypes.c_int(rows),
                                ctypes.c_int(Hl), ctypes.c_int(H), ctypes.c_int(1 if rms else 0), ctypes.c_int(mode),
                                ctypes.c_int(0), ctypes.c_int(0), ctypes.c_int(0), _lib.stream_ptr())
        _lib.check(st, "axb_add_norm_bwd")

    for i in range(n):
        bwd(i, 1)
    total = sums[0] + sums[1]
    for i in range(n):
        sums[i].copy_(total)
        bwd(i, 2)
    torch.cuda.synchronize()
    yr.backward(dy.float())
    dx = torch.cat(dxs, 1)
    _close(dx, hr.grad + dres.float(), 2e-2)
    _close(torch.cat([d[0] for d in dgbs]), gr.grad, 2e-2, 5e-2)
    if not rms:
        _close(torch.cat([d[1] for d in dgbs]), br.grad, 2e-2, 5e-2)
