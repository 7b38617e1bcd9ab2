"""Mamba kernels (causal conv1d, selective scan) against plain fp32 PyTorch references of the same ops."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _dev():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    return torch.device("cuda")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width,packed,strided", [(4, False, False), (4, True, True), (3, True, False), (2, False, True)])
def test_conv1d_fwd_bwd(dtype, width, packed, strided):
    from archscale_b200.ops.conv1d import causal_conv1d, causal_conv1d_ref
    dev = _dev()
    torch.manual_seed(0)
    B, L, C = 2, 203, 264
    wide = torch.randn(B, L, 2 * C, device=dev, dtype=dtype)
    x = (wide[..., :C] if strided else wide[..., :C].contiguous()).detach().requires_grad_(True)
    w = (torch.randn(C, width, device=dev) * 0.5).requires_grad_(True)
    b = torch.randn(C, device=dev).requires_grad_(True)
    seq_idx = None
    if packed:
        cuts = torch.tensor([0, 37, 38, 120, L], device=dev)
        seq_idx = (torch.arange(L, device=dev).view(1, L) >= cuts[1:-1].view(-1, 1)).sum(0).to(torch.int32).expand(B, L).contiguous()
    y = causal_conv1d(x, w, b, seq_idx=seq_idx, activation="silu", channel_last=True)
    g = torch.randn_like(y)
    y.backward(g)
    xr = x.detach().float().requires_grad_(True)
    wr, br = w.detach().clone().requires_grad_(True), b.detach().clone().requires_grad_(True)
    yr = causal_conv1d_ref(xr.transpose(1, 2), wr, br, seq_idx, "silu").transpose(1, 2)
    yr.backward(g.float())
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    assert torch.allclose(y.float(), yr, atol=tol, rtol=tol)
    assert torch.allclose(x.grad.float(), xr.grad, atol=tol, rtol=tol)
    scale = wr.grad.abs().max().item()
    assert (w.grad - wr.grad).abs().max().item() <= (1e-4 if dtype == torch.float32 else 2e-2) * scale
    assert (b.grad - br.grad).abs().max().item() <= (1e-4 if dtype == torch.float32 else 2e-2) * br.grad.abs().max().item()


@pytest.mark.parametrize("L,packed,with_z", [(64, False, True), (150, True, True), (257, True, False), (40, False, False)])
def test_selective_scan_fp32(L, packed, with_z):
    from archscale_b200.ops.selective_scan import selective_scan, selective_scan_ref
    dev = _dev()
    torch.manual_seed(1)
    B, Di, N = (1 if packed else 2), 48, 16
    mk = lambda *s: torch.randn(*s, device=dev)
    u, delta = mk(B, L, Di).requires_grad_(True), (mk(B, L, Di) * 0.5).requires_grad_(True)
    xdbl = mk(B, L, 2 * N + 8)
    Bm, Cm = xdbl[..., 8:8 + N].detach().requires_grad_(True), xdbl[..., 8 + N:].detach().requires_grad_(True)
    z = mk(B, L, Di).requires_grad_(True) if with_z else None
    A = (-torch.exp(torch.rand(Di, N, device=dev) * 2 - 1)).requires_grad_(True)
    D, bias = mk(Di).requires_grad_(True), (mk(Di) * 0.3).requires_grad_(True)
    cu = torch.tensor([0, 13, 64, 65, 130, L], device=dev, dtype=torch.int32) if packed else None
    y = selective_scan(u, delta, A, Bm, Cm, D, z=z, delta_bias=bias, delta_softplus=True, cu_seqlens=cu, channel_last=True)
    g = torch.randn_like(y)
    y.backward(g)
    leaves = [u, delta, A, Bm, Cm, D, bias] + ([z] if with_z else [])
    refs = [t.detach().clone().requires_grad_(True) for t in leaves]
    ur, dr, Ar, Br, Cr, Dr, br = refs[:7]
    zr = refs[7] if with_z else None
    t = lambda v: None if v is None else v.transpose(1, 2)
    yr = selective_scan_ref(t(ur), t(dr), Ar, t(Br), t(Cr), Dr, z=t(zr), delta_bias=br, delta_softplus=True,
                            cu_seqlens=cu).transpose(1, 2)
    yr.backward(g)
    assert torch.allclose(y, yr, atol=2e-4, rtol=2e-4), (y - yr).abs().max()
    for name, a, r in zip(["u", "delta", "A", "B", "C", "D", "bias", "z"], leaves, refs):
        err = (a.grad - r.grad).abs().max().item()
        assert err <= 2e-3 * max(1.0, r.grad.abs().max().item()), (name, err)


def test_selective_scan_bf16_strided_matches_fp32_oracle():
    from archscale_b200.ops.selective_scan import selective_scan, selective_scan_ref
    dev = _dev()
    torch.manual_seed(2)
    B, L, Di, N = 2, 300, 64, 16
    xz = torch.randn(B, L, 2 * Di, device=dev, dtype=torch.bfloat16)
    u, z = xz[..., :Di], xz[..., Di:]
    delta = (torch.randn(B, L, Di, device=dev) * 0.5).bfloat16()
    Bm, Cm = torch.randn(B, L, N, device=dev).bfloat16(), torch.randn(B, L, N, device=dev).bfloat16()
    A = -torch.exp(torch.rand(Di, N, device=dev))
    D, bias = torch.randn(Di, device=dev), torch.randn(Di, device=dev) * 0.3
    y = selective_scan(u, delta, A, Bm, Cm, D, z=z, delta_bias=bias, delta_softplus=True, channel_last=True)
    t = lambda v: v.float().transpose(1, 2)
    yr = selective_scan_ref(t(u), t(delta), A, t(Bm), t(Cm), D, z=t(z), delta_bias=bias, delta_softplus=True).transpose(1, 2)
    assert (y.float() - yr).abs().max().item() <= 2e-2 * max(1.0, yr.abs().max().item())


def test_mamba_block_runs_on_kernels():
    """A Mamba mixer forward+backward must go through the conv and scan kernels (launch counter moves)."""
    from archscale_b200.models.mamba import Mamba
    from archscale_b200.ops import backend
    dev = _dev()
    torch.manual_seed(3)
    m = Mamba(128, device=dev, dtype=torch.bfloat16)
    m.reset_parameters()
    x = torch.randn(2, 96, 128, device=dev, dtype=torch.bfloat16, requires_grad=True)
    before = backend.launches()
    out, _ = m(x)
    out.float().square().mean().backward()
    assert backend.launches() - before >= 4
    assert torch.isfinite(out.float()).all() and torch.isfinite(x.grad.float()).all()
    assert m.A_log.grad is not None and torch.isfinite(m.A_log.grad).all()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,cols", [(257, 2560), (64, 512), (1000, 1032)])
def test_layernorm_kernel(dtype, rows, cols):
    from archscale_b200.ops.norm import layer_norm, layer_norm_ref
    dev = _dev()
    torch.manual_seed(4)
    x = (torch.randn(rows, cols, device=dev) * 2 + 0.5).to(dtype).requires_grad_(True)
    w = torch.randn(cols, device=dev).requires_grad_(True)
    b = torch.randn(cols, device=dev).requires_grad_(True)
    y = layer_norm(x, w, b, 1e-5)
    g = torch.randn_like(y)
    y.backward(g)
    xr, wr, br = x.detach().float().requires_grad_(True), w.detach().clone().requires_grad_(True), b.detach().clone().requires_grad_(True)
    yr = layer_norm_ref(xr, wr, br, 1e-5)
    yr.backward(g.float())
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    assert torch.allclose(y.float(), yr, atol=tol, rtol=tol)
    assert torch.allclose(x.grad.float(), xr.grad, atol=tol * 4, rtol=tol * 4)
    for a, r in ((w.grad, wr.grad), (b.grad, br.grad)):
        assert (a - r).abs().max().item() <= (2e-4 if dtype == torch.float32 else 2e-2) * max(1.0, r.abs().max().item())


def test_optimizer_kernels_match_torch():
    """Fused Muon momentum and the segmented hyperball kernels of csrc/optim.cu against the foreach formulation."""
    from archscale_b200.ops import backend
    dev = _dev()
    ext = backend.require_extension()
    torch.manual_seed(5)
    n = 3 * 4096 + 1000 * 4
    g, m = torch.randn(n, device=dev), torch.randn(n, device=dev)
    u = torch.empty(n, device=dev, dtype=torch.bfloat16)
    m_ref = 0.95 * m + g * 0.5
    u_ref = (g * 0.5 + 0.95 * m_ref).bfloat16()
    ext.muon_momentum_(g, m, u, 0.95, True, torch.tensor(0.5, device=dev))
    assert torch.allclose(m, m_ref, atol=1e-6) and torch.equal(u, u_ref)
    # segments with boundaries inside a block and inside a warp's 128-element span
    cuts = [0, 1000, 1000 + 4100, 1000 + 4100 + 36, 9000, n]
    kidx = [4, 0, 2, 1, 3]
    bounds = torch.tensor(cuts, dtype=torch.int64, device=dev)
    kt = torch.tensor(kidx, dtype=torch.int32, device=dev)
    x = torch.randn(n, device=dev)
    acc = torch.zeros(6, device=dev)
    ext.seg_update_(0, x, None, bounds, kt, None, acc)
    want = torch.zeros(6, device=dev)
    for (a, b), k in zip(zip(cuts[:-1], cuts[1:]), kidx):
        want[k] = x[a:b].double().pow(2).sum().float()
    assert torch.allclose(acc, want, rtol=1e-4)
    coef = torch.rand(6, device=dev)
    x_ref = x.clone()
    for (a, b), k in zip(zip(cuts[:-1], cuts[1:]), kidx):
        x_ref[a:b] -= coef[k] * u[a:b].float()
    acc.zero_()
    ext.seg_update_(1, x, u, bounds, kt, coef, acc)
    assert torch.allclose(x, x_ref, atol=1e-6)
    for (a, b), k in zip(zip(cuts[:-1], cuts[1:]), kidx):
        want[k] = x_ref[a:b].double().pow(2).sum().float()
    assert torch.allclose(acc, want, rtol=1e-4)
    ext.seg_update_(2, x, None, bounds, kt, coef, None)
    for (a, b), k in zip(zip(cuts[:-1], cuts[1:]), kidx):
        x_ref[a:b] *= coef[k]
    assert torch.allclose(x, x_ref, atol=1e-6)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("cols,gsize,nbg,with_z", [(512, None, True, True), (512, 128, False, True), (1024, 256, True, False),
                                                    (2048, None, False, True)])
def test_gated_rmsnorm_kernel(dtype, cols, gsize, nbg, with_z):
    from archscale_b200.ops.norm import gated_rms_norm, gated_rms_norm_ref
    dev = _dev()
    torch.manual_seed(6)
    rows = 300
    x = torch.randn(rows, cols, device=dev).to(dtype).requires_grad_(True)
    z = torch.randn(rows, cols, device=dev).to(dtype).requires_grad_(True) if with_z else None
    w = (torch.rand(cols, device=dev) + 0.5).requires_grad_(True)
    y = gated_rms_norm(x, w, z, 1e-5, gsize, nbg)
    g = torch.randn_like(y)
    y.backward(g)
    xr = x.detach().float().requires_grad_(True)
    zr = z.detach().float().requires_grad_(True) if with_z else None
    wr = w.detach().clone().requires_grad_(True)
    yr = gated_rms_norm_ref(xr, wr, zr, 1e-5, gsize, nbg)
    yr.backward(g.float())
    tol = 3e-5 if dtype == torch.float32 else 4e-2
    assert torch.allclose(y.float(), yr, atol=tol, rtol=tol)
    assert torch.allclose(x.grad.float(), xr.grad, atol=tol * 4, rtol=tol * 4)
    if with_z:
        assert torch.allclose(z.grad.float(), zr.grad, atol=tol * 4, rtol=tol * 4)
    assert (w.grad - wr.grad).abs().max().item() <= (3e-4 if dtype == torch.float32 else 3e-2) * max(1.0, wr.grad.abs().max().item())


@pytest.mark.parametrize("W", [128, 256])
def test_diff_combine_kernel(W):
    from archscale_b200.ops.diff_attn import diff_combine, diff_combine_ref
    dev = _dev()
    torch.manual_seed(7)
    a1 = torch.randn(2, 70, 5, W, device=dev).bfloat16().requires_grad_(True)
    a2 = torch.randn(2, 70, 5, W, device=dev).bfloat16().requires_grad_(True)
    lam = torch.tensor(0.37, device=dev).bfloat16().requires_grad_(True)
    w = (torch.rand(W, device=dev) + 0.5).requires_grad_(True)
    y = diff_combine(a1, a2, lam, w, 0.8)
    g = torch.randn_like(y)
    y.backward(g)
    r = [t.detach().float().requires_grad_(True) for t in (a1, a2, lam, w)]
    yr = diff_combine_ref(r[0], r[1], r[2], r[3], 0.8)
    yr.backward(g.float())
    assert torch.allclose(y.float(), yr, atol=3e-2, rtol=3e-2)
    for got, ref in ((a1.grad, r[0].grad), (a2.grad, r[1].grad)):
        assert torch.allclose(got.float(), ref, atol=5e-2, rtol=5e-2)
    assert abs(float(lam.grad) - float(r[2].grad)) <= 3e-2 * max(1.0, abs(float(r[2].grad)))
    assert (w.grad - r[3].grad).abs().max().item() <= 3e-2 * max(1.0, r[3].grad.abs().max().item())
