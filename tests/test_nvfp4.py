"""NVFP4 (e2m1 elements, E4M3 scale per 16, fp32 scale per tensor): the PyTorch restatement on CPU, and the sm_100a
quantisers / block-scaled GEMM against it on a GPU."""
import pytest
import torch

from archscale_b200.ops import nvfp4
from archscale_b200.ops.mxfp8 import chunk_scales_ref, unchunk_scales_ref


def _rel(a, b):
    return float((a.float() - b.float()).norm() / (b.float().norm() + 1e-12))


def test_quantize_ref_values_lie_on_the_e2m1_grid_and_error_is_bounded():
    torch.manual_seed(0)
    x = torch.randn(64, 256) * torch.logspace(-2, 1, 64).unsqueeze(1)       # rows of very different magnitude
    q, sb, ts = nvfp4.quantize_ref(x)
    assert q.shape == (64, 128) and sb.shape == (64, 16) and ts.shape == (1,)
    xq = nvfp4.dequantize_ref(q, sb, ts)
    blocks = (xq.view(64, 16, 16) / (sb.view(torch.float8_e4m3fn).float() * ts).unsqueeze(-1).clamp_min(1e-30)).abs()
    grid = torch.tensor(nvfp4._GRID)
    assert (blocks.unsqueeze(-1) - grid).abs().amin(-1).max() < 1e-5
    # the largest element of a block is reproduced to within the scale's own rounding (E4M3: 2^-4 relative) plus half a step
    amax = x.view(64, 16, 16).abs().amax(-1)
    err = (xq - x).view(64, 16, 16).abs().amax(-1)
    assert bool((err <= 0.30 * amax + 1e-12).all())
    assert _rel(xq, x) < 0.12
    z = torch.zeros(16, 32)
    qz, sz, tz = nvfp4.quantize_ref(z)
    assert float(tz) == 1.0 and int(qz.max()) == 0 and torch.equal(nvfp4.dequantize_ref(qz, sz, tz), z)


def test_stochastic_rounding_is_unbiased():
    g = torch.Generator().manual_seed(1)
    x = torch.full((256, 16), 1.2)
    x[:, 0] = 6.0                                      # pins the block scale so that 1.2 sits between 1.0 and 1.5
    acc = torch.zeros_like(x)
    for _ in range(200):
        acc += nvfp4.fake_quantize(x, stochastic=True, generator=g)
    mean = (acc / 200)[:, 1:].mean()
    assert abs(float(mean) - 1.2) < 0.01
    assert float(nvfp4.fake_quantize(x)[0, 1]) == 1.0   # nearest rounding always lands on 1.0


def test_random_hadamard_keeps_products():
    torch.manual_seed(2)
    a, b = torch.randn(8, 64), torch.randn(5, 64)
    s = nvfp4._rht_sign("cpu")
    assert torch.allclose(nvfp4.random_hadamard(a, s) @ nvfp4.random_hadamard(b, s).t(), a @ b.t(), atol=1e-4)


@pytest.mark.parametrize("stochastic,rht", [(False, False), (True, True)])
def test_emulated_linear_forward_backward_close_to_fp32(stochastic, rht):
    torch.manual_seed(3)
    x = torch.randn(4, 32, 64, requires_grad=True)
    w = (torch.randn(48, 64) * 0.1).requires_grad_()
    b = torch.zeros(48, requires_grad=True)
    y = nvfp4.linear_nvfp4_emulated(x, w, b, stochastic=stochastic, rht=rht)
    g = torch.randn_like(y)
    y.backward(g)
    xr, wr, br = (t.detach().clone().requires_grad_() for t in (x, w, b))
    yr = torch.nn.functional.linear(xr, wr, br)
    yr.backward(g)
    assert _rel(y, yr) < 0.2 and _rel(x.grad, xr.grad) < 0.25 and _rel(w.grad, wr.grad) < 0.25
    assert torch.allclose(b.grad, br.grad, atol=1e-5)


def test_linear_module_flag_and_apply_nvfp4():
    from archscale_b200.models.layers import Linear, apply_nvfp4
    torch.manual_seed(4)
    net = torch.nn.Sequential(Linear(256, 512, bias=False), Linear(512, 100, bias=False))
    assert apply_nvfp4(net) == 1 and net[0].nvfp4 and not net[1].nvfp4
    x = torch.randn(32, 256)
    y = net[0](x)
    ref = x @ net[0].weight.t()
    assert 1e-4 < _rel(y, ref) < 0.2                    # quantised, and close


def test_scale_chunk_order_roundtrip_with_16_element_blocks():
    sb = torch.randint(0, 255, (200, 32), dtype=torch.uint8)      # 200 rows, K = 512
    assert torch.equal(unchunk_scales_ref(chunk_scales_ref(sb), 200, 32 * 32), sb)


# ------------------------------------------------------------------------------------------------ GPU
@pytest.mark.gpu
@pytest.mark.parametrize("R,C", [(256, 512), (512, 1024)])
def test_kernel_quantisers_match_the_restatement_bit_for_bit(R, C):
    torch.manual_seed(5)
    x = (torch.randn(R, C, device="cuda") * torch.logspace(-1, 1, R, device="cuda").unsqueeze(1)).bfloat16()
    x[3, 32:48] = 0                                     # an all-zero block
    q, sf, am = nvfp4.quantize(x)
    qr, sbr, tsr = nvfp4.quantize_ref(x)
    assert torch.equal(am, nvfp4.tensor_amax(x)) and torch.equal(nvfp4.scale_from_amax(am), tsr)
    assert torch.equal(q, qr)
    assert torch.equal(unchunk_scales_ref(sf, R, C * 2), sbr)       # K/16 scale columns = (2K)/32
    qt, sft, _ = nvfp4.quantize(x, colwise=True)
    qtr, sbtr, _ = nvfp4.quantize_ref(x.t().contiguous(), ts=tsr)
    assert torch.equal(qt, qtr)
    assert torch.equal(unchunk_scales_ref(sft, C, R * 2), sbtr)
    (q2, sf2, _), (qt2, sft2, _) = nvfp4.quantize_both(x)           # one read, both orientations
    assert torch.equal(q2, q) and torch.equal(sf2, sf) and torch.equal(qt2, qt) and torch.equal(sft2, sft)
    assert float(nvfp4.amax(torch.zeros(256, 256, device="cuda", dtype=torch.bfloat16))) == 0.0


@pytest.mark.gpu
@pytest.mark.parametrize("M,N,K", [(256, 256, 256), (512, 384, 1024), (300, 520, 512), (128, 8192, 256)])
def test_block_scaled_fp4_gemm_matches_dequantised_matmul(M, N, K):
    from archscale_b200.ops import backend
    torch.manual_seed(6)
    a = torch.randn(M, K, device="cuda").bfloat16()
    b = (torch.randn(N, K, device="cuda") * 0.3).bfloat16()
    qa, qb = nvfp4.quantize(a), nvfp4.quantize(b)
    out = nvfp4.gemm(qa, qb, out_f32=True)
    torch.cuda.synchronize()
    assert backend.require_extension().device_status() == 0
    ar = nvfp4.dequantize_ref(*nvfp4.quantize_ref(a))
    br = nvfp4.dequantize_ref(*nvfp4.quantize_ref(b))
    ref = (ar.double() @ br.double().t()).float()
    assert _rel(out, ref) < 1e-4
    acc = torch.ones(M, N, device="cuda")
    nvfp4.gemm(qa, qb, acc=acc, alpha=0.5)
    assert _rel(acc, 1 + 0.5 * ref) < 1e-4


@pytest.mark.gpu
def test_kernel_stochastic_rounding_is_unbiased_and_stays_on_neighbouring_grid_values():
    x = torch.full((256, 256), 1.2, device="cuda").bfloat16()
    x[:, ::16] = 6.0                                   # pins every block scale so that 1.2 sits between 1.0 and 1.5
    acc = torch.zeros(256, 256, device="cuda")
    first = None
    for _ in range(64):
        q, sf, am = nvfp4.quantize(x, stochastic=True)
        d = nvfp4.dequantize_ref(q, unchunk_scales_ref(sf, 256, 512), nvfp4.scale_from_amax(am))
        first = d if first is None else first
        acc += d
    body = torch.ones(256, 256, dtype=torch.bool, device="cuda")
    body[:, ::16] = False
    vals = torch.unique(first[body])
    assert set(round(float(v), 4) for v in vals) <= {1.0, 1.5}            # only the two neighbours of 1.2 (bf16: 1.203)
    mean = float((acc / 64)[body].mean())
    assert abs(mean - float(x[0, 1])) < 0.01
    assert torch.equal(first[~body], torch.full_like(first[~body], 6.0))


@pytest.mark.gpu
def test_kernel_hadamard_transform_cancels_in_the_product():
    """(dyᵀ·D·H)(xᵀ·D·H)ᵀ = dyᵀ·x: the transformed transposed operands give the same weight gradient up to quantisation."""
    torch.manual_seed(8)
    T, N, K = 512, 256, 256
    dy = torch.randn(T, N, device="cuda").bfloat16()
    x = torch.randn(T, K, device="cuda").bfloat16()
    x[5, 7] = 40.0                                     # an outlier that the transform spreads over its block
    ref = dy.float().t() @ x.float()
    plain = nvfp4.gemm(nvfp4.quantize(dy, colwise=True), nvfp4.quantize(x, colwise=True), out_f32=True)
    rht = nvfp4.gemm(nvfp4.quantize(dy, colwise=True, rht=True), nvfp4.quantize(x, colwise=True, rht=True), out_f32=True)
    assert _rel(plain, ref) < 0.2 and _rel(rht, ref) < 0.2
    # the kernel's transform equals the restatement's: dequantised transposed operand against fake-quantised H-transformed xᵀ
    qt, sft, am4 = nvfp4.quantize(x, colwise=True, rht=True)
    got = nvfp4.dequantize_ref(qt, unchunk_scales_ref(sft, K, 2 * T), nvfp4.scale_from_amax(am4))
    want = nvfp4.random_hadamard(x.float().t().contiguous(), nvfp4._rht_sign("cuda"))
    assert _rel(got, want) < 0.15


@pytest.mark.gpu
def test_nvfp4_linear_kernel_path_matches_emulation(monkeypatch):
    monkeypatch.setenv("ARCHSCALE_B200_NVFP4_SR", "0")
    monkeypatch.setenv("ARCHSCALE_B200_NVFP4_RHT", "0")
    torch.manual_seed(7)
    x = torch.randn(2, 256, 512, device="cuda").bfloat16().requires_grad_()
    w = (torch.randn(768, 512, device="cuda") * 0.05).bfloat16().requires_grad_()
    y = nvfp4.linear_nvfp4(x, w)
    g = torch.randn_like(y)
    y.backward(g)
    xe, we = (t.detach().clone().requires_grad_() for t in (x, w))
    ye = nvfp4.linear_nvfp4_emulated(xe, we, None, stochastic=False, rht=False)
    ye.backward(g)
    assert _rel(y, ye) < 1e-2 and _rel(x.grad, xe.grad) < 1e-2 and _rel(w.grad, we.grad) < 1e-2
    xr, wr = (t.detach().float().requires_grad_() for t in (x, w))
    yr = torch.nn.functional.linear(xr, wr)
    yr.backward(g.float())
    assert _rel(y, yr) < 0.2 and _rel(x.grad, xr.grad) < 0.25 and _rel(w.grad, wr.grad) < 0.25


@pytest.mark.gpu
def test_nvfp4_linear_with_stochastic_rounding_and_hadamard_close_to_fp32():
    torch.manual_seed(9)
    x = torch.randn(2, 256, 512, device="cuda").bfloat16().requires_grad_()
    w = (torch.randn(768, 512, device="cuda") * 0.05).bfloat16().requires_grad_()
    y = nvfp4.linear_nvfp4(x, w)                       # both options on by default
    g = torch.randn_like(y)
    y.backward(g)
    xr, wr = (t.detach().float().requires_grad_() for t in (x, w))
    yr = torch.nn.functional.linear(xr, wr)
    yr.backward(g.float())
    assert _rel(y, yr) < 0.2 and _rel(x.grad, xr.grad) < 0.3 and _rel(w.grad, wr.grad) < 0.3
