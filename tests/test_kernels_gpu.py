"""sm_100a kernels against plain PyTorch fp32 references of the same operation."""

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
@pytest.mark.parametrize("shape", [(512, 2048), (333, 1024), (64, 4096), (1000, 256), (5003, 2048), (2501, 3072)])
def test_norm_fwd_bwd(rms, shape):
    from axonn_b200 import ops

    torch.manual_seed(0)
    rows, H = shape
    x = torch.randn(rows, H, device=DEV).bfloat16().requires_grad_(True)
    g = (1 + 0.1 * torch.randn(H, device=DEV)).bfloat16().requires_grad_(True)
    b = (0.1 * torch.randn(H, device=DEV)).bfloat16().requires_grad_(True)
    dy = torch.randn(rows, H, device=DEV).bfloat16()
    y = ops.rms_norm(x, g, 1e-5) if rms else ops.layer_norm(x, g, b, 1e-5)
    y.backward(dy)
    xr, gr, br = (t.detach().float().requires_grad_(True) for t in (x, g, b))
    if rms:
        yr = xr * torch.rsqrt(xr.pow(2).mean(-1, keepdim=True) + 1e-5) * gr
    else:
        yr = F.layer_norm(xr, (H,), gr, br, 1e-5)
    yr.backward(dy.float())
    _close(y, yr, 1e-2)
    _close(x.grad, xr.grad, 2e-2)
    _close(g.grad, gr.grad, 2e-2, 5e-2)
    if not rms:
        _close(b.grad, br.grad, 2e-2, 5e-2)


@pytest.mark.parametrize("rms", [False, True])
def test_norm_forward_split_hidden_modes(rms):
    """The three launches of a norm whose hidden dimension is split over ranks, emulated on one GPU: partial row sums
    per slice (mode 1), their sum (what the all-reduce produces), then the finishing mode (3), which turns the sums
    into (mean, rstd) in place and applies them to the slice."""
    import ctypes

    from axonn_b200.ops import _lib

    torch.manual_seed(4)
    rows, H, n = 257, 2048, 2
    x = torch.randn(rows, H, device=DEV).bfloat16()
    g = (1 + 0.1 * torch.randn(H, device=DEV)).bfloat16()
    b = (0.1 * torch.randn(H, device=DEV)).bfloat16()
    L = _lib.lib()
    Hl = H // n
    xs = [x[:, i * Hl:(i + 1) * Hl].contiguous() for i in range(n)]
    ys = [torch.empty_like(t) for t in xs]
    stats = [torch.empty(rows, 2, dtype=torch.float32, device=DEV) for _ in range(n)]

    def call(i, mode):
        gi, bi = g[i * Hl:(i + 1) * Hl].contiguous(), b[i * Hl:(i + 1) * Hl].contiguous()
        st = L.axb_norm_fwd(_lib.ptr(xs[i]), _lib.ptr(gi), _lib.ptr(None if rms else bi), _lib.ptr(ys[i]),
                            _lib.ptr(stats[i]), ctypes.c_int(rows), ctypes.c_int(Hl), ctypes.c_int(H),
                            ctypes.c_float(1e-5), ctypes.c_int(1 if rms else 0), ctypes.c_int(mode), ctypes.c_int(0),
                            ctypes.c_int(0), _lib.stream_ptr())
        _lib.check(st, "axb_norm_fwd")

    for i in range(n):
        call(i, 1)
    total = stats[0] + stats[1]
    for i in range(n):
        stats[i].copy_(total)
        call(i, 3)
    y = torch.cat(ys, 1)
    xr = x.float()
    if rms:
        ref = xr * torch.rsqrt(xr.pow(2).mean(-1, keepdim=True) + 1e-5) * g.float()
        mean_ref = torch.zeros(rows, device=DEV)
    else:
        ref = F.layer_norm(xr, (H,), g.float(), b.float(), 1e-5)
        mean_ref = xr.mean(-1)
    _close(y, ref, 1e-2)
    assert (stats[0][:, 0] - mean_ref).abs().max().item() < 1e-3        # (mean, rstd) left behind for the backward
    assert torch.equal(stats[0], stats[1])


@pytest.mark.parametrize("rms", [False, True])
@pytest.mark.parametrize("shape", [(300, 2048), (64, 4096), (130, 1024), (17, 8192)])
def test_add_norm_fused_residual(rms, shape):
    """h = x + delta and norm(h) in one kernel, backward with the residual-path gradient added in the kernel:
    against the two plain steps evaluated in fp32."""
    from axonn_b200 import ops

    rows, H = shape
    torch.manual_seed(5)
    x = torch.randn(rows, H, device=DEV).bfloat16().requires_grad_(True)
    dl = torch.randn(rows, H, device=DEV).bfloat16().requires_grad_(True)
    g = (1 + 0.1 * torch.randn(H, device=DEV)).bfloat16().requires_grad_(True)
    b = (0.1 * torch.randn(H, device=DEV)).bfloat16().requires_grad_(True)
    dy = torch.randn(rows, H, device=DEV).bfloat16()
    dh = torch.randn(rows, H, device=DEV).bfloat16()
    h, y = ops.add_rms_norm(x, dl, g, 1e-5) if rms else ops.add_layer_norm(x, dl, g, b, 1e-5)
    torch.autograd.backward([h, y], [dh, dy])
    assert torch.equal(h, (x.detach() + dl.detach()))          # the same rounding as a separate add
    xr, dr, gr, br = (t.detach().float().requires_grad_(True) for t in (x, dl, g, b))
    hr = (xr + dr) + ((xr + dr).bfloat16().float() - (xr + dr)).detach()   # value rounded like the kernel, gradient of the sum
    if rms:
        yr = hr * torch.rsqrt(hr.pow(2).mean(-1, keepdim=True) + 1e-5) * gr
    else:
        yr = F.layer_norm(hr, (H,), gr, br, 1e-5)
    torch.autograd.backward([hr, yr], [dh.float(), dy.float()])
    _close(y, yr, 1e-2)
    _close(x.grad, xr.grad, 2e-2)
    assert torch.equal(x.grad, dl.grad)
    _close(g.grad, gr.grad, 2e-2, 5e-2)
    if not rms:
        _close(b.grad, br.grad, 2e-2, 5e-2)


def test_gelu_swiglu():
    from axonn_b200 import ops
    from axonn_b200.ops.activation import _split_gu

    torch.manual_seed(1)
    x = torch.randn(257, 1024, device=DEV).bfloat16().requires_grad_(True)
    dy = torch.randn_like(x)
    y = ops.gelu(x)
    y.backward(dy)
    xr = x.detach().float().requires_grad_(True)
    yr = F.gelu(xr, approximate="tanh")
    yr.backward(dy.float())
    _close(y, yr, 1e-2)
    _close(x.grad, xr.grad, 1e-2)

    gu = torch.randn(130, 2 * 512, device=DEV).bfloat16().requires_grad_(True)
    do = torch.randn(130, 512, device=DEV).bfloat16()
    o = ops.swiglu(gu)
    o.backward(do)
    gur = gu.detach().float().requires_grad_(True)
    gg, uu = _split_gu(gur)
    orf = F.silu(gg) * uu
    orf.backward(do.float())
    _close(o, orf, 1e-2)
    _close(gu.grad, gur.grad, 1e-2)


def test_rope_matches_reference_and_inverts():
    from axonn_b200 import ops
    from axonn_b200.ops.rope import _rope_torch

    torch.manual_seed(2)
    B, S, G, n, D = 2, 96, 3, 4, 128
    table = ops.rope_table(S, D, 500000.0, torch.device(DEV))
    qkv = torch.randn(B, S, G, n + 2, D, device=DEV).bfloat16()
    ref = _rope_torch(qkv[:, :, :, : n + 1].float().cpu(), table.cpu(), False)
    src = qkv.clone().requires_grad_(True)
    work = src * 1.0
    ops.apply_rope(work[:, :, :, : n + 1], table)
    _close(work[:, :, :, : n + 1].cpu(), ref, 1e-2)
    assert torch.equal(work[:, :, :, n + 1], qkv[:, :, :, n + 1])  # v untouched
    # backward is the inverse rotation
    gout = torch.randn_like(work)
    work.backward(gout)
    gref = gout.clone().float().cpu()
    gref[:, :, :, : n + 1] = _rope_torch(gref[:, :, :, : n + 1], table.cpu(), True)
    _close(src.grad.cpu(), gref, 1e-2)
    # 4-D form
    q = torch.randn(B, S, 8, 64, device=DEV).bfloat16()
    t64 = ops.rope_table(S, 64, 10000.0, torch.device(DEV))
    r4 = _rope_torch(q.float().cpu(), t64.cpu(), False)
    q2 = (q * 1.0)
    from axonn_b200.ops.rope import _rope_apply
    _rope_apply(q2, t64, False)
    _close(q2.cpu(), r4, 1e-2)


@pytest.mark.parametrize("V", [512, 50304 // 2])
def test_cross_entropy(V):
    from axonn_b200 import ops

    torch.manual_seed(3)
    rows = 300
    z = (torch.randn(rows, V, device=DEV) * 2).bfloat16()
    t = torch.randint(0, V, (rows,), device=DEV)
    t[5] = -100
    zr = z.float().requires_grad_(True)
    lr = F.cross_entropy(zr, t, ignore_index=-100)
    lr.backward()
    zz = z.clone().requires_grad_(True)
    zin = zz * 1.0
    loss = ops.cross_entropy(zin, t)
    loss.backward()
    assert abs(loss.item() - lr.item()) < 2e-3 * abs(lr.item())
    _close(zz.grad, zr.grad, 2e-2, 1e-5)


def test_fused_adamw_matches_torch():
    from axonn_b200.optim import FusedAdamW

    torch.manual_seed(4)
    shapes = [(1000,), (257, 33), (70000,), (8,)]
    ps = [torch.randn(s, device=DEV).bfloat16().requires_grad_(True) for s in shapes]
    ref = [p.detach().float().clone().requires_grad_(True) for p in ps]
    opt = FusedAdamW(ps, lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    ropt = torch.optim.AdamW(ref, lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    for _ in range(4):
        for p, r in zip(ps, ref):
            g = torch.randn_like(r)
            p.grad = g.bfloat16()
            r.grad = g.bfloat16().float()
        opt.step()
        ropt.step()
    for p, r in zip(ps, ref):
        _close(opt.state[p]["master"], r, 1e-5, 1e-6)
        _close(p, r, 1e-2)


def test_multi_tensor_norm_and_scale():
    from axonn_b200 import ops

    torch.manual_seed(5)
    ts = [torch.randn(n, device=DEV).to(dt) for n, dt in
          [(100000, torch.bfloat16), (7, torch.float32), (65537, torch.float32), (131072, torch.bfloat16)]]
    got = ops.multi_tensor_l2norm_sq(ts).item()
    want = sum(t.float().pow(2).sum().item() for t in ts)
    assert abs(got - want) <= 1e-4 * want
    before = [t.clone() for t in ts]
    ops.multi_tensor_scale_(ts, 0.5)
    for a, b in zip(ts, before):
        _close(a, b.float() * 0.5, 1e-2, 1e-6)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_fused_sgd_matches_torch_sgd(dtype):
    from axonn_b200.optim import FusedSGD

    torch.manual_seed(9)
    shapes = [(1000, 33), (4096,), (257, 129), (70000,)]
    ours = [torch.nn.Parameter(torch.randn(s, device=DEV).to(dtype)) for s in shapes]
    ref = [torch.nn.Parameter(p.detach().float().clone()) for p in ours]
    a = FusedSGD(ours, lr=0.05, momentum=0.9, weight_decay=0.01)
    b = torch.optim.SGD(ref, lr=0.05, momentum=0.9, weight_decay=0.01)
    for _ in range(3):
        for p, q in zip(ours, ref):
            g = torch.randn_like(q)
            p.grad = g.to(dtype)
            q.grad = g.to(dtype).float()
        a.step()
        b.step()
    for p, q in zip(ours, ref):
        _close(p.detach(), q.detach(), 1e-2 if dtype == torch.bfloat16 else 1e-5, 1e-5)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("n", [4096, 1_000_003, 14336 * 512])
def test_prune_topk(dtype, n):
    from axonn_b200 import ops

    torch.manual_seed(6)
    g = torch.randn(n, device=DEV).to(dtype)
    k = max(1, int(round(n * 0.1)))
    ref = g.clone()
    thr = ref.abs().float().kthvalue(n - k + 1).values
    ref = ref * (ref.abs().float() >= thr).to(dtype)
    out = ops.prune_topk_(g.clone(), 0.1)
    assert torch.equal(out, ref), f"kept {(out != 0).sum().item()} vs {(ref != 0).sum().item()}"


@pytest.mark.parametrize("cfg", [(2, 256, 2, 1, 128), (1, 512, 2, 4, 128), (2, 384, 3, 1, 64), (1, 1024, 1, 2, 64)])
def test_flash_attention_forward(cfg):
    from axonn_b200.ops import _lib
    from axonn_b200.ops.attention_cuda import flash_fwd_packed

    B, S, G, qpk, D = cfg
    torch.manual_seed(7)
    qkv = torch.randn(B, S, G, qpk + 2, D, device=DEV).bfloat16()
    scale = D ** -0.5
    out, lse = flash_fwd_packed(qkv, scale)
    torch.cuda.synchronize()
    assert _lib.lib().axb_device_status(0, 1) == 0
    q = qkv[:, :, :, :qpk].reshape(B, S, G * qpk, D).float().transpose(1, 2)
    k = qkv[:, :, :, qpk].float().transpose(1, 2).repeat_interleave(qpk, dim=1)
    v = qkv[:, :, :, qpk + 1].float().transpose(1, 2).repeat_interleave(qpk, dim=1)
    s = (q @ k.transpose(-1, -2)) * scale
    mask = torch.ones(S, S, device=DEV, dtype=torch.bool).tril()
    s = s.masked_fill(~mask, float("-inf"))
    ref = (s.softmax(-1) @ v).transpose(1, 2)
    _close(out, ref, 2e-2, 2e-2)
    lse_ref = torch.logsumexp(s, -1)
    assert (lse - lse_ref).abs().max().item() < 2e-2


@pytest.mark.parametrize("D", [128, 64])
def test_flash_attention_forward_large_scores(D):
    """Scores whose row maximum keeps growing by far more than 2^8 from one KV tile to the next: the two-tile
    forward must rescale its tensor-memory accumulator (it only does so past that threshold), and rows whose
    maximum moves by less must stay exact although their reference maximum is stale."""
    from axonn_b200.ops import _lib
    from axonn_b200.ops.attention_cuda import flash_fwd_packed

    B, S, G, qpk = 1, 1024, 2, 2
    torch.manual_seed(8)
    qkv = torch.randn(B, S, G, qpk + 2, D, device=DEV)
    ramp = torch.linspace(0.2, 4.0, S, device=DEV)[None, :, None, None]
    qkv[:, :, :, qpk] *= ramp                     # later keys score higher and higher
    qkv[:, :, :, :qpk] *= 2.0
    qkv = qkv.bfloat16()
    scale = D ** -0.5
    out, lse = flash_fwd_packed(qkv, scale)
    torch.cuda.synchronize()
    assert _lib.lib().axb_device_status(0, 1) == 0
    q = qkv[:, :, :, :qpk].reshape(B, S, G * qpk, D).float().transpose(1, 2)
    k = qkv[:, :, :, qpk].float().transpose(1, 2).repeat_interleave(qpk, dim=1)
    v = qkv[:, :, :, qpk + 1].float().transpose(1, 2).repeat_interleave(qpk, dim=1)
    s = (q @ k.transpose(-1, -2)) * scale
    s = s.masked_fill(~torch.ones(S, S, device=DEV, dtype=torch.bool).tril(), float("-inf"))
    ref = (s.softmax(-1) @ v).transpose(1, 2)
    assert torch.isfinite(out.float()).all()
    _close(out, ref, 2e-2, 2e-2)
    assert (lse - torch.logsumexp(s, -1)).abs().max().item() < 5e-2


@pytest.mark.parametrize("mode", ["fused", "split"])
@pytest.mark.parametrize("cfg", [(2, 256, 2, 1, 128), (1, 512, 2, 4, 128), (2, 384, 3, 1, 64), (1, 640, 1, 2, 64),
                                 (1, 1024, 1, 2, 64)])
def test_flash_attention_backward(cfg, mode, monkeypatch):
    """Both backward implementations (one kernel with an fp32 dQ accumulator; two kernels without atomics) against
    autograd through an fp32 reference; the head_dim 64 GQA cases have many short steps per work item, which is
    where an ordering mistake between the softmax warps of a row shows first."""
    from axonn_b200.ops import _lib
    from axonn_b200.ops.attention_cuda import flash_bwd_packed, flash_fwd_packed

    monkeypatch.setenv("AXONN_FA_BWD", mode)
    B, S, G, qpk, D = cfg
    torch.manual_seed(11)
    qkv = torch.randn(B, S, G, qpk + 2, D, device=DEV).bfloat16()
    d_out = torch.randn(B, S, G * qpk, D, device=DEV).bfloat16()
    scale = D ** -0.5
    out, lse = flash_fwd_packed(qkv, scale)
    dqkv = flash_bwd_packed(qkv, out, d_out, lse, scale)
    torch.cuda.synchronize()
    assert _lib.lib().axb_device_status(0, 1) == 0
    x = qkv.float().requires_grad_(True)
    q = x[:, :, :, :qpk].reshape(B, S, G * qpk, D).transpose(1, 2)
    k = x[:, :, :, qpk].transpose(1, 2).repeat_interleave(qpk, dim=1)
    v = x[:, :, :, qpk + 1].transpose(1, 2).repeat_interleave(qpk, dim=1)
    s = (q @ k.transpose(-1, -2)) * scale
    mask = torch.ones(S, S, device=DEV, dtype=torch.bool).tril()
    ref = (s.masked_fill(~mask, float("-inf")).softmax(-1) @ v).transpose(1, 2)
    ref.backward(d_out.float())
    for name, sl in (("dq", slice(0, qpk)), ("dk", slice(qpk, qpk + 1)), ("dv", slice(qpk + 1, qpk + 2))):
        got, want = dqkv[:, :, :, sl].float(), x.grad[:, :, :, sl]
        err = (got - want).abs().max().item()
        assert err <= 3e-2 * want.abs().max().item() + 2e-2, f"{name}: {err} vs {want.abs().max().item()}"


@pytest.mark.parametrize("shape", [(16384, 2048), (1000, 136), (7, 8), (4099, 6144)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_column_sum(shape, dtype):
    from axonn_b200 import ops

    torch.manual_seed(3)
    x = torch.randn(*shape, device=DEV).to(dtype)
    got = ops.column_sum(x)
    ref = x.double().sum(0)
    assert got.dtype == torch.float32
    err = (got.double() - ref).abs().max().item()
    assert err <= 1e-4 * shape[0] ** 0.5 + 1e-3 * ref.abs().max().item(), err


def test_gelu_backward_colsum():
    from axonn_b200 import ops

    torch.manual_seed(4)
    x = torch.randn(4099, 1032, device=DEV).bfloat16()
    dy = torch.randn_like(x)
    dx, cs = ops.gelu_backward_colsum(dy, x)
    ref = ops.gelu_backward(dy, x)
    assert torch.equal(dx, ref)
    # the kernel sums the unrounded products: compare with an fp32 evaluation, not with the bf16 dx
    exact = ops.gelu_backward(dy.float().cpu(), x.float().cpu()).sum(0)
    _close(cs.cpu(), exact, 1e-3, 5e-2)
