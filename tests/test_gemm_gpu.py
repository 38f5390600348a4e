"""tcgen05 GEMM against a plain PyTorch fp32 reference of the same product."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(layout, a, b):
    a, b = a.float(), b.float()
    if layout == "nt":
        return a @ b.t()
    if layout == "nn":
        return a @ b
    return a.t() @ b


def _operands(layout, M, N, K, dtype, dev):
    g = torch.Generator(device=dev).manual_seed(M * 7 + N * 3 + K)
    sa = (M, K) if layout != "tn" else (K, M)
    sb = (N, K) if layout == "nt" else (K, N)
    a = (torch.randn(sa, device=dev, generator=g) * 0.5).to(dtype)
    b = (torch.randn(sb, device=dev, generator=g) * 0.5).to(dtype)
    return a, b


SHAPES = [
    (128, 128, 64), (128, 256, 128), (256, 512, 256), (384, 640, 192),
    (200, 136, 72),            # ragged M, N, K (multiples of 8 only)
    (1024, 1024, 1024), (4096, 2048, 512), (520, 2056, 1032),
]


@pytest.mark.parametrize("layout", ["nt", "nn", "tn"])
@pytest.mark.parametrize("shape", SHAPES)
def test_gemm_matches_fp32_reference(layout, shape):
    from axonn_b200 import ops
    from axonn_b200.ops import _lib

    M, N, K = shape
    dev = torch.device("cuda", 0)
    a, b = _operands(layout, M, N, K, torch.bfloat16, dev)
    fn = {"nt": ops.matmul_nt, "nn": ops.matmul_nn, "tn": ops.matmul_tn}[layout]
    out = fn(a, b)
    torch.cuda.synchronize()
    assert _lib.lib().axb_device_status(0, 1) == 0
    ref = _ref(layout, a, b)
    err = (out.float() - ref).abs().max().item()
    scale = ref.abs().max().item()
    assert err <= 1e-2 * scale + 1e-2, f"{layout} {shape}: max err {err} (scale {scale})"
    # fp32 output: only accumulation-order differences remain
    out32 = fn(a, b, out_dtype=torch.float32)
    torch.cuda.synchronize()
    err32 = (out32 - ref).abs().max().item()
    assert err32 <= 2e-4 * scale + 1e-4, f"{layout} {shape}: fp32-out max err {err32}"


def test_gemm_fp16_and_accumulate():
    from axonn_b200 import ops

    dev = torch.device("cuda", 0)
    a, b = _operands("nt", 512, 384, 256, torch.float16, dev)
    out = ops.matmul_nt(a, b, out_dtype=torch.float32)
    ref = _ref("nt", a, b)
    assert (out - ref).abs().max().item() <= 2e-3 * ref.abs().max().item()
    acc = torch.ones_like(out)
    ops.matmul_nt(a, b, out=acc, accumulate=True)
    assert (acc - (ref + 1)).abs().max().item() <= 2e-3 * ref.abs().max().item()
    a, b = _operands("tn", 256, 512, 1024, torch.bfloat16, dev)
    acc = torch.full((256, 512), 2.0, device=dev)
    ops.matmul_tn(a, b, out=acc, accumulate=True)
    ref = _ref("tn", a, b) + 2
    assert (acc - ref).abs().max().item() <= 2e-4 * ref.abs().max().item() + 1e-4


def test_gemm_bias_gelu_epilogue():
    from axonn_b200 import ops

    dev = torch.device("cuda", 0)
    a, b = _operands("nt", 384, 512, 256, torch.bfloat16, dev)
    bias = (torch.randn(512, device=dev) * 0.5).bfloat16()
    z_ref = _ref("nt", a, b) + bias.float()
    out = ops.matmul_nt(a, b, bias=bias, epilogue=ops.EPI_BIAS)
    assert (out.float() - z_ref).abs().max().item() <= 1e-2 * z_ref.abs().max().item() + 1e-2
    aux = torch.empty(384, 512, device=dev, dtype=torch.bfloat16)
    out = ops.matmul_nt(a, b, bias=bias, epilogue=ops.EPI_BIAS_GELU, aux=aux)
    g_ref = torch.nn.functional.gelu(z_ref, approximate="tanh")
    assert (aux.float() - z_ref).abs().max().item() <= 1e-2 * z_ref.abs().max().item() + 1e-2
    assert (out.float() - g_ref).abs().max().item() <= 1e-2 * g_ref.abs().max().item() + 1e-2


@pytest.mark.parametrize("layout", ["nt", "nn", "tn"])
def test_gemm_cta_pair_path_ragged(layout):
    """Shapes wide enough for the CTA-pair (256x256 tile) kernel: odd number of 128-row tiles, ragged N and K."""
    from axonn_b200 import ops
    from axonn_b200.ops import _lib

    M, N, K = 4104, 4360, 520
    dev = torch.device("cuda", 0)
    a, b = _operands(layout, M, N, K, torch.bfloat16, dev)
    fn = {"nt": ops.matmul_nt, "nn": ops.matmul_nn, "tn": ops.matmul_tn}[layout]
    ref = _ref(layout, a, b)
    scale = ref.abs().max().item()
    for _ in range(2):
        out32 = fn(a, b, out_dtype=torch.float32)
    torch.cuda.synchronize()
    assert _lib.lib().axb_device_status(0, 1) == 0
    assert (out32 - ref).abs().max().item() <= 2e-4 * scale + 1e-4
    acc = torch.full((M, N), 3.0, device=dev)
    fn(a, b, out=acc, accumulate=True)
    assert (acc - (ref + 3)).abs().max().item() <= 2e-4 * scale + 1e-4


def test_gemm_cta_pair_path_epilogue():
    from axonn_b200 import ops

    dev = torch.device("cuda", 0)
    M, N, K = 8192, 4096, 1024
    a, b = _operands("nt", M, N, K, torch.bfloat16, dev)
    bias = (torch.randn(N, device=dev) * 0.5).bfloat16()
    z_ref = _ref("nt", a, b) + bias.float()
    aux = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
    out = ops.matmul_nt(a, b, bias=bias, epilogue=ops.EPI_BIAS_GELU, aux=aux)
    g_ref = torch.nn.functional.gelu(z_ref, approximate="tanh")
    assert (aux.float() - z_ref).abs().max().item() <= 1e-2 * z_ref.abs().max().item() + 1e-2
    assert (out.float() - g_ref).abs().max().item() <= 1e-2 * g_ref.abs().max().item() + 1e-2


@pytest.mark.gpu
@pytest.mark.parametrize("shape", [(1024, 512, 256), (4096, 4096, 1024), (300, 136, 64)])
def test_fused_all_reduce_loopback(shape):
    """Two-rank GEMM+all-reduce emulated on one GPU (peer slots aliased to local memory): 2 * A B^T."""
    from axonn_b200.parallel import fused

    M, N, K = shape
    torch.manual_seed(0)
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    bias = torch.randn(N, device="cuda", dtype=torch.bfloat16)
    ref = 2.0 * (a.float() @ b.float().t()) + bias.float()
    for _ in range(3):   # three calls: both parities of the double-buffered inbox and the done handshake
        out = fused.gemm_all_reduce_loopback(a, b, bias=bias, epilogue=1)
    torch.cuda.synchronize()
    err = (out.float() - ref).abs().max() / ref.abs().max()
    assert err < 2e-2, err


@pytest.mark.gpu
@pytest.mark.parametrize("shape", [(1024, 512, 256), (8192, 4096, 512), (300, 136, 64)])
def test_fused_two_shot_all_reduce_loopback(shape):
    """Two-shot protocol emulated on one GPU as rank 0 of 2: the 32-row units this rank owns (even index) hold
    2 * A B^T + bias both in the local result and in the buffer that stands in for the peer's C; the kernel's
    mailbox, owner-only pushes, row-wise reducer and end-of-call wait all run."""
    from axonn_b200.ops import _lib
    from axonn_b200.parallel import fused

    M, N, K = shape
    torch.manual_seed(0)
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    bias = torch.randn(N, device="cuda", dtype=torch.bfloat16)
    ref = 2.0 * (a.float() @ b.float().t()) + bias.float()
    for _ in range(3):
        out, peer = fused.gemm_all_reduce_loopback(a, b, bias=bias, epilogue=1, two_shot=True)
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    rows = torch.arange(M, device="cuda")
    owned = ((rows // 32) % 2) == 0
    scale = ref.abs().max()
    assert (out.float()[owned] - ref[owned]).abs().max() < 2e-2 * scale
    assert torch.equal(out[owned], peer[owned])


def test_silent_peer_times_out_and_context_survives():
    """A peer that never raises its flags: the bounded wait of the fused kernel runs out, the kernel returns,
    the status word names the reason, and the next (healthy) call on the same buffers is correct."""
    from axonn_b200.ops import _lib
    from axonn_b200.parallel import fused

    torch.manual_seed(1)
    a = torch.randn(512, 256, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(512, 256, device="cuda", dtype=torch.bfloat16)
    ref = 2.0 * (a.float() @ b.float().t())
    fused.gemm_all_reduce_loopback(a, b)             # healthy call first
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    _lib.set_wait_timeout_ms(50)
    try:
        fused.gemm_all_reduce_loopback(a, b, silent_peer=True)
        torch.cuda.synchronize()
        st = _lib.device_status()
        # the watcher (0x121 / 0x123) or the reducer warps waiting for it (0x120 / 0x122) run out first
        assert st in (0x120, 0x121, 0x122, 0x123), hex(st)
        with pytest.raises(_lib.KernelError):
            fused.gemm_all_reduce_loopback(a, b, silent_peer=True)
            torch.cuda.synchronize()
            _lib.check_status()
    finally:
        _lib.set_wait_timeout_ms(2000)
    for _ in range(2):
        out = fused.gemm_all_reduce_loopback(a, b)
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    assert (out.float() - ref).abs().max() <= 2e-2 * ref.abs().max()


@pytest.mark.parametrize("shape", [(4, 256, 512, 256), (3, 640, 1024, 320), (2, 2560, 2048, 1024), (8, 128, 264, 192)])
def test_batched_gemm_matches_fp32(shape):
    """All three layouts of the batched CTA-pair GEMM (one launch over the tiles of E problems) against fp32
    matmuls; M and N need not be multiples of the tile, so tiles run into the next problem's rows and must not
    store them."""
    from axonn_b200.ops import gemm
    from axonn_b200.ops import _lib

    E, M, N, K = shape
    torch.manual_seed(21)
    a = torch.randn(E, M, K, device="cuda:0").bfloat16()
    b = torch.randn(E, N, K, device="cuda:0").bfloat16()
    y = gemm.bmm_nt(a, b)
    ref = torch.matmul(a.float(), b.float().transpose(1, 2))
    assert (y.float() - ref).abs().max().item() <= 2e-2 * ref.abs().max().item()
    g = torch.randn(E, M, N, device="cuda:0").bfloat16()
    if N % 64 == 0:
        gx = gemm.bmm_nn(g, b)                       # [E, M, N] @ [E, N, K]
        ref = torch.matmul(g.float(), b.float())
        assert (gx.float() - ref).abs().max().item() <= 2e-2 * ref.abs().max().item()
    if M % 64 == 0:
        gw = gemm.bmm_tn(g, a, out_dtype=torch.float32)   # [E, M, N].T @ [E, M, K]
        ref = torch.matmul(g.float().transpose(1, 2), a.float())
        assert (gw - ref).abs().max().item() <= 2e-2 * ref.abs().max().item()
    torch.cuda.synchronize()
    assert _lib.device_status() == 0


@pytest.mark.parametrize("shape", [(2, 4, 640, 512, 256), (1, 8, 2560, 1024, 512), (3, 2, 192, 264, 128)])
def test_batched_gemm_row_mask(shape):
    """Capacity-padded problems: only the first ``seg[e, s]`` rows of every segment hold data, the rest are zero.
    With the mask the kernels skip tiles (K blocks for the weight gradient) without data; the results must equal
    the unmasked products, zeros included."""
    from axonn_b200.ops import _lib, gemm

    E, nseg, seg_rows, N, K = shape
    M = nseg * seg_rows
    torch.manual_seed(22)
    seg = torch.randint(0, seg_rows + 1, (E, nseg), device="cuda:0", dtype=torch.int32)
    seg[0, 0] = 0
    seg[-1, -1] = seg_rows
    rows = torch.arange(M, device="cuda:0") % seg_rows
    live = rows[None, :] < seg.long().repeat_interleave(seg_rows, dim=1)          # [E, M]
    a = torch.randn(E, M, K, device="cuda:0").bfloat16() * live[:, :, None]
    b = torch.randn(E, N, K, device="cuda:0").bfloat16()
    y = gemm.bmm_nt(a, b, seg=seg, seg_rows=seg_rows)
    ref = torch.matmul(a.float(), b.float().transpose(1, 2))
    assert (y.float() - ref).abs().max().item() <= 2e-2 * ref.abs().max().item()
    assert (y.float()[~live] == 0).all()
    g = torch.randn(E, M, N, device="cuda:0").bfloat16() * live[:, :, None]
    if N % 64 == 0:
        gx = gemm.bmm_nn(g, b, seg=seg, seg_rows=seg_rows)
        ref = torch.matmul(g.float(), b.float())
        assert (gx.float() - ref).abs().max().item() <= 2e-2 * ref.abs().max().item()
    if M % 64 == 0:
        gw = gemm.bmm_tn(g, a, out_dtype=torch.float32, seg=seg, seg_rows=seg_rows)
        ref = torch.matmul(g.float().transpose(1, 2), a.float())
        assert (gw - ref).abs().max().item() <= 2e-2 * max(ref.abs().max().item(), 1.0)
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
