"""sm_100a kernels vs plain PyTorch fp32 oracles (run on a B200)."""
import math

import pytest
import torch

from archscale_b200 import ops
from archscale_b200.ops import backend

pytestmark = pytest.mark.gpu


def _ext():
    return backend.require_extension()


def _rel(a, b):
    return (a.float() - b.float()).norm() / (b.float().norm() + 1e-12)


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 512), (200, 264, 136), (1024, 2048, 2048), (8, 8, 64),
                                   (4096, 1024, 264)])
@pytest.mark.parametrize("mode", [0, 1, 2])
def test_gemm_bf16_layouts(M, N, K, mode):
    torch.manual_seed(0)
    dev = "cuda"
    A = torch.randn(M, K, device=dev) * 0.5
    B = torch.randn(N, K, device=dev) * 0.5
    ref = A @ B.t()
    a = A.bfloat16() if mode != 2 else A.t().contiguous().bfloat16()          # mode 2 stores Aᵀ: [K, M]
    b = B.bfloat16() if mode == 0 else B.t().contiguous().bfloat16()          # modes 1, 2 store [K, N]
    ref = (a.float() if mode != 2 else a.float().t()) @ (b.float().t() if mode == 0 else b.float())
    out = _ext().gemm_bf16(a, b, mode, torch.bfloat16, None)
    torch.cuda.synchronize()
    assert _ext().device_status() == 0
    assert out.shape == (M, N)
    assert _rel(out, ref) < 1e-2, float(_rel(out, ref))


def test_gemm_fp32_accumulate_and_epilogue():
    torch.manual_seed(1)
    M, N, K = 384, 520, 320
    a = (torch.randn(K, M, device="cuda") * 0.3).bfloat16()
    b = (torch.randn(K, N, device="cuda") * 0.3).bfloat16()
    acc = torch.randn(M, N, device="cuda")
    ref = acc + a.float().t() @ b.float()
    _ext().gemm_bf16(a, b, 2, torch.float32, acc)
    assert _rel(acc, ref) < 1e-3
    x = (torch.randn(M, K, device="cuda") * 0.3).bfloat16()
    w = (torch.randn(N, K, device="cuda") * 0.3).bfloat16()
    c = torch.randn(M, N, device="cuda").bfloat16()
    out = _ext().gemm_bf16_epi(x, w, 0, 0.5, -2.0, c)
    ref = 0.5 * (x.float() @ w.float().t()) - 2.0 * c.float()
    assert _rel(out, ref) < 1e-2
    assert _ext().device_status() == 0


def test_linear_autograd_matches_reference():
    torch.manual_seed(2)
    x = (torch.randn(4, 96, 256, device="cuda")).bfloat16().requires_grad_()
    w = (torch.randn(512, 256, device="cuda") * 0.05).bfloat16().requires_grad_()
    bias = torch.randn(512, device="cuda").bfloat16().requires_grad_()
    y = ops.linear(x, w, bias)
    g = torch.randn_like(y)
    y.backward(g)
    xr, wr, br = (t.detach().float().requires_grad_() for t in (x, w, bias))
    yr = torch.nn.functional.linear(xr, wr, br)
    yr.backward(g.float())
    assert _rel(y, yr) < 1e-2 and _rel(x.grad, xr.grad) < 1e-2 and _rel(w.grad, wr.grad) < 1e-2 and _rel(bias.grad, br.grad) < 1e-2


@pytest.mark.parametrize("rows,cols", [(64, 256), (1000, 2048), (37, 1024), (300, 1984), (129, 3080)])
@pytest.mark.parametrize("xdt,odt", [(torch.float32, torch.bfloat16), (torch.bfloat16, torch.bfloat16), (torch.float32, torch.float32)])
def test_rmsnorm(rows, cols, xdt, odt):
    torch.manual_seed(3)
    x = torch.randn(rows, cols, device="cuda").to(xdt).requires_grad_()
    w = (1 + 0.1 * torch.randn(cols, device="cuda")).requires_grad_()
    y = ops.rms_norm(x, w, 1e-5, out_dtype=odt)
    assert y.dtype == odt
    g = torch.randn(rows, cols, device="cuda").to(odt)
    y.backward(g)
    xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    yr = ops.rms_norm_ref(xr, wr, 1e-5)
    yr.backward(g.float())
    tol = 2e-2 if (xdt == torch.bfloat16 or odt == torch.bfloat16) else 1e-5
    assert _rel(y, yr) < tol and _rel(x.grad, xr.grad) < tol and _rel(w.grad, wr.grad) < tol


def test_rmsnorm_no_weight():
    x = torch.randn(100, 512, device="cuda").requires_grad_()
    y = ops.rms_norm(x, None, 1e-5)
    y.sum().backward()
    xr = x.detach().clone().requires_grad_()
    ops.rms_norm_ref(xr, None, 1e-5).sum().backward()
    assert _rel(x.grad, xr.grad) < 1e-4


def test_swiglu_both_forms():
    torch.manual_seed(4)
    x = torch.randn(300, 2 * 704, device="cuda").bfloat16().requires_grad_()
    y = ops.swiglu_packed(x)
    g = torch.randn_like(y)
    y.backward(g)
    xr = x.detach().float().requires_grad_()
    a, b = xr.chunk(2, dim=-1)
    yr = torch.nn.functional.silu(a) * b
    yr.backward(g.float())
    assert _rel(y, yr) < 1e-2 and _rel(x.grad, xr.grad) < 1e-2
    p = torch.randn(64, 256, device="cuda").bfloat16().requires_grad_()
    q = torch.randn(64, 256, device="cuda").bfloat16().requires_grad_()
    z = ops.swiglu(p, q)
    z.backward(torch.ones_like(z))
    pr, qr = p.detach().float().requires_grad_(), q.detach().float().requires_grad_()
    (torch.nn.functional.silu(pr) * qr).sum().backward()
    assert _rel(p.grad, pr.grad) < 1e-2 and _rel(q.grad, qr.grad) < 1e-2


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("ls,zs", [(0.0, 0.0), (0.1, 1e-4)])
def test_cross_entropy_kernel(dtype, ls, zs):
    torch.manual_seed(5)
    rows, V = 77, 32000
    logits = (torch.randn(rows, V, device="cuda") * 2).to(dtype)
    tgt = torch.randint(0, V, (rows,), device="cuda")
    tgt[5] = -100
    lr = logits.detach().float().requires_grad_()
    loss_ref = ops.cross_entropy_ref(lr, tgt, -100, ls, zs, reduction="sum")
    loss_ref.backward()
    work = logits.clone()
    loss = _ext().cross_entropy_fwd_bwd_(work, tgt, -100, ls, zs)
    assert abs(float(loss.sum()) - float(loss_ref)) / abs(float(loss_ref)) < 1e-3
    assert _rel(work, lr.grad) < (2e-2 if dtype == torch.bfloat16 else 1e-4)


def test_fused_linear_cross_entropy_matches_reference():
    torch.manual_seed(6)
    N, H, V = 1024, 256, 4096
    x = (torch.randn(N, H, device="cuda") * 0.5).bfloat16().requires_grad_()
    w = (torch.randn(V, H, device="cuda") * 0.05).bfloat16().requires_grad_()
    t = torch.randint(0, V, (N,), device="cuda")
    loss = ops.fused_linear_cross_entropy(x, w, t, chunk_rows=256)
    loss.backward()
    xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    lr = ops.fused_linear_cross_entropy_ref(xr, wr, t)
    lr.backward()
    assert abs(float(loss) - float(lr)) < 2e-2
    assert _rel(x.grad, xr.grad) < 3e-2 and _rel(w.grad, wr.grad) < 3e-2


@pytest.mark.parametrize("D,H,G", [(128, 4, 2), (64, 6, 3)])
@pytest.mark.parametrize("use_norm,use_rope", [(True, True), (False, True), (True, False)])
def test_qknorm_rope(D, H, G, use_norm, use_rope):
    torch.manual_seed(7)
    B, T = 2, 50
    q = torch.randn(B, T, H, D, device="cuda").bfloat16().requires_grad_()
    k = torch.randn(B, T, G, D, device="cuda").bfloat16().requires_grad_()
    qw = (1 + 0.1 * torch.randn(D, device="cuda")).requires_grad_() if use_norm else None
    kw = (1 + 0.1 * torch.randn(D, device="cuda")).requires_grad_() if use_norm else None
    cos, sin = ops.build_rope_cache(T, D, torch.bfloat16, "cuda") if use_rope else (None, None)
    qo, ko = ops.qk_norm_rope(q, k, qw, kw, cos, sin, 1e-5)
    gq, gk = torch.randn_like(qo), torch.randn_like(ko)
    (qo.float() * gq.float()).sum().backward(retain_graph=True)
    (ko.float() * gk.float()).sum().backward()
    from archscale_b200.ops.rope import qk_norm_rope_ref
    qr, kr = q.detach().float().requires_grad_(), k.detach().float().requires_grad_()
    qwr = qw.detach().clone().requires_grad_() if use_norm else None
    kwr = kw.detach().clone().requires_grad_() if use_norm else None
    qro, kro = qk_norm_rope_ref(qr, kr, qwr, kwr, cos, sin, 1e-5)
    ((qro * gq.float()).sum() + (kro * gk.float()).sum()).backward()
    assert _rel(qo, qro) < 2e-2 and _rel(ko, kro) < 2e-2
    assert _rel(q.grad, qr.grad) < 2e-2 and _rel(k.grad, kr.grad) < 2e-2
    if use_norm:
        assert _rel(qw.grad, qwr.grad) < 2e-2 and _rel(kw.grad, kwr.grad) < 2e-2


def test_newton_schulz_cuda_close_to_reference():
    torch.manual_seed(8)
    G = torch.randn(512, 1024, device="cuda")
    O = ops.newton_schulz(G)
    R = ops.newton_schulz_ref(G)
    assert _rel(O, R) < 0.1
    s = torch.linalg.svdvals(O.float())
    assert s.max() < 1.6 and s.min() > 0.3


@pytest.mark.parametrize("cols", [1024, 2048, 2560, 1984, 520, 3592])
@pytest.mark.parametrize("res_dtype", [torch.float32, torch.bfloat16])
def test_add_rms_norm_fused(cols, res_dtype):
    torch.manual_seed(9)
    rows = 517
    res = torch.randn(rows, cols, device="cuda").to(res_dtype).requires_grad_()
    h = torch.randn(rows, cols, device="cuda").bfloat16().requires_grad_()
    w = (1 + 0.1 * torch.randn(cols, device="cuda")).requires_grad_()
    x, n = ops.add_rms_norm(res, h, w, 1e-5, 0.25)
    gx, gn = torch.randn_like(x), torch.randn_like(n)
    torch.autograd.backward((x, n), (gx, gn))
    rr, hr, wr = (t.detach().float().requires_grad_() for t in (res, h, w))
    xr, nr = ops.add_rms_norm_ref(rr, hr, wr, 1e-5, 0.25, torch.float32)
    torch.autograd.backward((xr, nr), (gx.float(), gn.float()))
    assert _rel(x, xr) < 1e-5 and _rel(n, nr) < 1e-2
    assert _rel(res.grad, rr.grad) < 1e-2 and _rel(h.grad, hr.grad) < 1e-2 and _rel(w.grad, wr.grad) < 1e-2
    # without a pending branch (first block): residual passes through unchanged
    x2, n2 = ops.add_rms_norm(res.detach(), None, w.detach(), 1e-5, 1.0)
    assert _rel(n2, ops.rms_norm_ref(res.detach().float(), w.detach(), 1e-5)) < 1e-2


@pytest.mark.parametrize("cols", [1024, 2048, 1984])
def test_add_rms_norm_fused_bf16_stream(cols):
    """Residual stream kept in bf16: x is the bf16-rounded sum, the norm and every gradient follow from that x."""
    torch.manual_seed(11)
    rows = 517
    res = torch.randn(rows, cols, device="cuda").bfloat16().requires_grad_()
    h = torch.randn(rows, cols, device="cuda").bfloat16().requires_grad_()
    w = (1 + 0.1 * torch.randn(cols, device="cuda")).requires_grad_()
    x, n = ops.add_rms_norm(res, h, w, 1e-5, 0.25, stream_dtype=torch.bfloat16)
    assert x.dtype == torch.bfloat16 and n.dtype == torch.bfloat16
    gx, gn = torch.randn_like(x), torch.randn_like(n)
    torch.autograd.backward((x, n), (gx, gn))
    assert res.grad.dtype == torch.bfloat16
    rr, hr, wr = (t.detach().float().requires_grad_() for t in (res, h, w))
    xr, nr = ops.add_rms_norm_ref(rr, hr, wr, 1e-5, 0.25, torch.float32, torch.float32)
    torch.autograd.backward((xr, nr), (gx.float(), gn.float()))
    assert torch.equal(x, xr.bfloat16())                          # the stream is the rounded fp32 sum
    assert _rel(n, nr) < 1e-2
    assert _rel(res.grad, rr.grad) < 1e-2 and _rel(h.grad, hr.grad) < 1e-2 and _rel(w.grad, wr.grad) < 1e-2
    x2, n2 = ops.add_rms_norm(res.detach(), None, w.detach(), 1e-5, 1.0, stream_dtype=torch.bfloat16)
    assert x2.dtype == torch.bfloat16 and _rel(n2, ops.rms_norm_ref(res.detach().float(), w.detach(), 1e-5)) < 1e-2


def test_model_deferred_residual_matches_generic_path():
    """The fused (deferred residual) block path and the generic module path give the same loss/grads."""
    from archscale_b200 import Config
    from archscale_b200.models.gpt import GPT
    torch.manual_seed(10)
    cfg = Config.from_name("transformer_gqa4_d8", n_layer=2, ar=None, n_embd=1024, n_head=8, n_query_groups=4,
                           head_dim=128, intermediate_size=2048, vocab_size=1024, padding_multiple=64, block_size=256,
                           qk_norm=True, depth_scale=True)
    with torch.device("cuda"):
        m = GPT(cfg)
    m.reset_parameters()
    m = m.bfloat16()
    idx = torch.randint(0, 1024, (2, 256), device="cuda")
    out = m(idx).logits
    out.float().pow(2).mean().backward()
    g1 = {n: p.grad.clone() for n, p in m.named_parameters()}
    m.zero_grad()
    import archscale_b200.ops.norm as nm
    saved = nm.fused_cols_ok
    nm.fused_cols_ok = lambda cols: False
    try:
        out2 = m(idx).logits
        out2.float().pow(2).mean().backward()
    finally:
        nm.fused_cols_ok = saved
    assert _rel(out, out2) < 2e-2
    for n, p in m.named_parameters():
        assert _rel(g1[n], p.grad) < 5e-2, n


@pytest.mark.parametrize("Bn,M,N,K,mode", [(5, 256, 256, 1024, 0), (3, 200, 136, 264, 0), (7, 256, 1024, 256, 1), (2, 384, 520, 136, 1)])
def test_gemm_batched(Bn, M, N, K, mode):
    torch.manual_seed(11)
    a = (torch.randn(Bn, M, K, device="cuda") * 0.3).bfloat16()
    b = (torch.randn(Bn, N, K, device="cuda") * 0.3).bfloat16() if mode == 0 else (torch.randn(Bn, K, N, device="cuda") * 0.3).bfloat16()
    c = torch.randn(Bn, M, N, device="cuda").bfloat16()
    out = _ext().gemm_bf16_batched(a, b, mode, 0.5, 2.0, c)
    ref = 0.5 * torch.bmm(a.float(), b.float().transpose(1, 2) if mode == 0 else b.float()) + 2.0 * c.float()
    torch.cuda.synchronize()
    assert _ext().device_status() == 0
    assert _rel(out, ref) < 1e-2


def test_newton_schulz_batched_matches_per_matrix():
    torch.manual_seed(12)
    G = torch.randn(6, 256, 1024, device="cuda")
    O = ops.newton_schulz(G)
    R = torch.stack([ops.newton_schulz(g) for g in G])
    assert _rel(O, R) < 2e-2
    Gt = torch.randn(4, 1024, 256, device="cuda")          # tall: Gram matrix XᵀX on the untransposed data (two-CTA kernel)
    Ot = ops.newton_schulz(Gt)
    assert _rel(Ot, ops.newton_schulz_ref(Gt)) < 0.1
    was = _ext().set_gemm_pair(False)                       # one-CTA kernel: transposed copy in and out
    try:
        Ot1 = ops.newton_schulz(Gt)
    finally:
        _ext().set_gemm_pair(was)
    assert _rel(Ot, Ot1) < 2e-2
    assert _ext().device_status() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("M,N,K", [(3072, 2048, 16384), (2048, 5632, 8192), (512, 512, 32768)])
@pytest.mark.parametrize("pair", [False, True])
def test_wgrad_split_k_accumulates_exactly_like_unsplit(M, N, K, pair):
    """Accumulating TN GEMM whose tile count fills the last wave badly: the serial split-K path must add the same
    products (fp32 accumulation, fixed order) as a reference matmul, on top of the existing contents, twice in a row."""
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    from archscale_b200.ops import backend
    ext = backend.require_extension()
    torch.manual_seed(0)
    a = (torch.randn(K, M, device="cuda") * 0.1).bfloat16()
    b = (torch.randn(K, N, device="cuda") * 0.1).bfloat16()
    acc = torch.ones(M, N, device="cuda")
    was = ext.set_gemm_pair(pair)           # both kernels split K (148 CTAs or 74 pairs to fill)
    try:
        ext.gemm_bf16(a, b, 2, torch.float32, acc)
        ext.gemm_bf16(a, b, 2, torch.float32, acc)
        torch.cuda.synchronize()
    finally:
        ext.set_gemm_pair(was)
    ref = 1.0 + 2.0 * (a.float().t() @ b.float())
    assert ext.device_status() == 0
    assert (acc - ref).abs().max().item() <= 2e-3 * ref.abs().max().item()


@pytest.mark.parametrize("pair", [False, True])
@pytest.mark.parametrize("M,N,K,mode", [(384, 520, 320, 2), (1000, 776, 264, 0), (640, 1288, 512, 1), (4096, 4096, 1024, 0)])
def test_gemm_one_cta_and_two_cta_kernels_agree_with_fp32(pair, M, N, K, mode):
    """Both GEMM kernels (128×256 tile per SM, 256×256 tile per SM pair) against an fp32 matmul, all three layouts,
    ragged edges, bf16 output and accumulating fp32 output."""
    from archscale_b200.ops import backend
    ext = backend.require_extension()
    torch.manual_seed(3)
    A = (torch.randn(M, K, device="cuda") * 0.3).bfloat16()
    B = (torch.randn(N, K, device="cuda") * 0.3).bfloat16()
    a = A if mode != 2 else A.t().contiguous()
    b = B if mode == 0 else B.t().contiguous()
    ref = A.float() @ B.float().t()
    was = ext.set_gemm_pair(pair)
    try:
        out = ext.gemm_bf16(a, b, mode, torch.bfloat16, None)
        acc = torch.full((M, N), 0.5, device="cuda")
        ext.gemm_bf16(a, b, mode, torch.float32, acc)
        torch.cuda.synchronize()
    finally:
        ext.set_gemm_pair(was)
    assert ext.device_status() == 0
    assert _rel(out, ref) < 1e-2
    assert _rel(acc, ref + 0.5) < 1e-3


@pytest.mark.gpu
@pytest.mark.parametrize("Bn,M,K", [(3, 640, 264), (2, 2048, 512), (5, 256, 1024)])
def test_batched_symmetric_product_matches_full_product(Bn, M, K):
    """X·Xᵀ and c·A·A + b·A computed from the upper triangle of tiles and mirrored (two-CTA kernel) equal the full products."""
    torch.manual_seed(12)
    x = (torch.randn(Bn, M, K, device="cuda") * 0.1).bfloat16()
    full = _ext().gemm_bf16_batched(x, x, 0, 1.0, 0.0, None, False)
    sym = _ext().gemm_bf16_batched(x, x, 0, 1.0, 0.0, None, True)
    ref = x.float() @ x.float().transpose(1, 2)
    assert _rel(sym, ref) < 1e-2 and _rel(full, ref) < 1e-2
    assert torch.equal(sym, sym.transpose(1, 2))
    a = sym.contiguous()
    poly = _ext().gemm_bf16_batched(a, a, 0, 0.7, -1.3, a, True)
    ref2 = 0.7 * (a.float() @ a.float()) - 1.3 * a.float()
    assert _rel(poly, ref2) < 1e-2
    torch.cuda.synchronize()
    assert _ext().device_status() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("mode", [0, 1, 2])
def test_batched_gemm_per_matrix_factors(mode):
    """alpha_vec / beta_vec multiply into alpha / beta per matrix of the batch (first Newton–Schulz iteration on unscaled data)."""
    torch.manual_seed(13)
    Bn, M, N, K = 4, 384, 512, 320
    a = (torch.randn(Bn, M, K, device="cuda") * 0.2).bfloat16()
    b = (torch.randn(Bn, N, K, device="cuda") * 0.2).bfloat16()
    c = torch.randn(Bn, M, N, device="cuda").bfloat16()
    av = torch.rand(Bn, device="cuda") + 0.5
    bv = torch.rand(Bn, device="cuda") - 0.5
    aa = a if mode != 2 else a.transpose(1, 2).contiguous()
    bb = b if mode == 0 else b.transpose(1, 2).contiguous()
    out = _ext().gemm_bf16_batched(aa, bb, mode, 0.5, 2.0, c, False, av, bv)
    ref = 0.5 * av.view(-1, 1, 1) * (a.float() @ b.float().transpose(1, 2)) + 2.0 * bv.view(-1, 1, 1) * c.float()
    torch.cuda.synchronize()
    assert _ext().device_status() == 0
    assert _rel(out, ref) < 1e-2


@pytest.mark.parametrize("mode", [0, 1])
def test_adamw_fused_matches_foreach(mode):
    """One-pass AdamW over a flat fp32 slice (with the gradient-clip coefficient folded in) against the foreach formulas."""
    from archscale_b200.optim import scalar_opts
    ext = backend.require_extension()
    torch.manual_seed(0)
    n = 1 << 18
    x = torch.randn(n, device="cuda")
    m, v = torch.randn(n, device="cuda") * 0.1, torch.rand(n, device="cuda") * 0.01
    g = torch.randn(n, device="cuda")
    scale = torch.tensor(0.37, device="cuda")
    xr, mr, vr = x.clone(), m.clone(), v.clone()
    lr, b1, b2, eps, wd, step = 3e-3, 0.9, 0.95, 1e-8, 0.1, 7
    if mode == 0:
        ext.adamw_fused_(0, x, g, m, v, None, lr, b1, b2, eps, wd, step, scale, None)
        scalar_opts.adamw_update_foreach([xr], [g * scale], [mr], [vr], lr, b1, b2, wd, step, eps)
        assert torch.allclose(x, xr, atol=1e-6, rtol=1e-5)
    else:
        u, acc = torch.empty_like(x), torch.zeros(2, device="cuda")
        ext.adamw_fused_(1, x, g, m, v, u, lr, b1, b2, eps, 0.0, step, scale, acc)
        ur = scalar_opts.adamw_direction_([mr], [vr], [g * scale], b1, b2, eps, step)[0]
        assert torch.equal(x, xr)                                   # mode 1 leaves the parameter alone
        assert torch.allclose(u, ur, atol=1e-5, rtol=1e-4)
        assert torch.allclose(acc, torch.stack([xr.pow(2).sum(), ur.pow(2).sum()]), rtol=1e-4)
    assert torch.allclose(m, mr, atol=1e-6) and torch.allclose(v, vr, atol=1e-7)


@pytest.mark.parametrize("M,I,K", [(512, 256, 256), (1000, 1408, 512), (4096, 5632, 2048), (264, 72, 136)])
def test_gemm_with_swiglu_epilogue_equals_gemm_then_swiglu(M, I, K):
    """The pre-activation is the plain GEMM's result bit for bit, and the activation is what the separate SwiGLU kernel
    makes of it (both computed from the bf16-rounded values); against fp32 PyTorch the usual bf16 tolerance holds."""
    torch.manual_seed(8)
    x = torch.randn(M, K, device="cuda").bfloat16()
    w = (torch.randn(2 * I, K, device="cuda") * 0.05).bfloat16()
    h, act = _ext().gemm_swiglu(x, w, True)
    h_ref = ops.matmul_nt(x, w)
    assert torch.equal(h, h_ref)
    assert torch.equal(act, _ext().swiglu_packed_fwd(h_ref))
    _, act_only = _ext().gemm_swiglu(x, w, False)
    assert torch.equal(act_only, act)
    hf = x.float() @ w.float().t()
    assert _rel(act, torch.nn.functional.silu(hf[:, :I]) * hf[:, I:]) < 2e-2
    assert _ext().device_status() == 0


def test_linear_swiglu_autograd_matches_reference():
    torch.manual_seed(9)
    x = torch.randn(4, 256, 512, device="cuda").bfloat16().requires_grad_()
    w = (torch.randn(2 * 1024, 512, device="cuda") * 0.05).bfloat16().requires_grad_()
    y = ops.linear_swiglu(x, w)
    assert y is not None and y.shape == (4, 256, 1024)
    g = torch.randn_like(y)
    y.backward(g)
    xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    hr = xr @ wr.t()
    yr = torch.nn.functional.silu(hr[..., :1024]) * hr[..., 1024:]
    yr.backward(g.float())
    assert _rel(y, yr) < 2e-2 and _rel(x.grad, xr.grad) < 3e-2 and _rel(w.grad, wr.grad) < 3e-2


@pytest.mark.parametrize("grouped", [True, False])
@pytest.mark.parametrize("G,qpk,D,norm,rope", [(4, 4, 128, True, True), (2, 5, 64, False, True), (3, 1, 128, True, False)])
def test_qkv_norm_rope_from_the_fused_projection_layout(G, qpk, D, norm, rope, grouped):
    """Norm + rotation read in place from the projection's layout (per group [q…, k, v], or blocked [q | k | v]) equal
    split → qk_norm_rope, values and gradients."""
    torch.manual_seed(12)
    B, T, H = 2, 96, G * qpk
    W = (H + 2 * G) * D
    pad = 40                                                 # a column slice of a wider matrix (e.g. a gate projection beside it)
    wide = torch.randn(B, T, W + pad, device="cuda").bfloat16().requires_grad_()
    qw = (1 + 0.1 * torch.randn(D, device="cuda")).requires_grad_() if norm else None
    kw = (1 + 0.1 * torch.randn(D, device="cuda")).requires_grad_() if norm else None
    cos, sin = (None, None)
    if rope:
        cos, sin = ops.build_rope_cache(T, D, torch.bfloat16, "cuda")

    def split(t):
        y = t[..., :W]
        if grouped:
            a, b, c = y.view(B, T, G, qpk + 2, D).split((qpk, 1, 1), dim=-2)
        else:
            a, b, c = y.split((H * D, G * D, G * D), dim=-1)
        return a.reshape(B, T, H, D), b.reshape(B, T, G, D), c.reshape(B, T, G, D)

    qkv = wide[..., :W]
    assert ops.qkv_norm_rope_supported(qkv, H, G, cos, qw)
    q, k, v = ops.qkv_norm_rope(qkv, H, G, grouped, qw, kw, cos, sin, 1e-5)
    gq, gk, gv = torch.randn_like(q), torch.randn_like(k), torch.randn_like(v)
    torch.autograd.backward((q, k, v), (gq, gk, gv))
    got = [wide.grad.clone()] + ([qw.grad.clone(), kw.grad.clone()] if norm else [])
    wide.grad = None
    if norm:
        qw.grad = kw.grad = None
    qs, ks, vs = split(wide)
    q2, k2 = ops.qk_norm_rope(qs, ks, qw, kw, cos, sin, 1e-5)
    torch.autograd.backward((q2, k2, vs), (gq, gk, gv))
    assert torch.equal(q, q2) and torch.equal(k, k2) and torch.equal(v, vs)
    assert torch.equal(got[0], wide.grad)
    if norm:
        assert _rel(got[1], qw.grad) < 1e-5 and _rel(got[2], kw.grad) < 1e-5
