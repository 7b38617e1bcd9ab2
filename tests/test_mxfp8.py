"""MXFP8: reference quantiser properties (CPU) and the sm_100a quantise / block-scaled GEMM kernels (GPU)."""
import pytest
import torch

from archscale_b200.ops import mxfp8


def test_reference_quantiser_never_saturates_and_roundtrips_scales():
    torch.manual_seed(0)
    x = torch.randn(256, 384) * torch.logspace(-3, 3, 384)
    q, e = mxfp8.quantize_ref(x)
    assert q.float().abs().max() <= 448
    deq = mxfp8.dequantize_ref(q, e)
    blk_amax = x.view(256, 12, 32).abs().amax(-1, keepdim=True).expand(256, 12, 32).reshape(256, 384)
    assert ((deq - x).abs() <= blk_amax * 2 ** -3).all()            # e4m3 has 3 mantissa bits
    sf = mxfp8.chunk_scales_ref(e)
    assert sf.numel() == 2 * 3 * 512
    assert torch.equal(mxfp8.unchunk_scales_ref(sf, 256, 384), e)
    # byte position of (row 37, block 6): chunk (0, 1), m0 = 5, m1 = 1, k1 = 2
    assert sf[(0 * 3 + 1) * 512 + 5 * 16 + 1 * 4 + 2] == e[37, 6]


@pytest.mark.gpu
@pytest.mark.parametrize("R,C", [(256, 384), (128, 128), (384, 1024)])
def test_quantise_kernels_match_reference(R, C):
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    torch.manual_seed(1)
    x = (torch.randn(R, C, device="cuda") * torch.logspace(-2, 2, C, device="cuda")).bfloat16()
    q, sf = mxfp8.quantize(x)
    qr, er = mxfp8.quantize_ref(x)
    assert torch.equal(mxfp8.unchunk_scales_ref(sf, R, C), er)
    assert torch.equal(q.view(torch.float8_e4m3fn).float(), qr.float())
    qt, sft = mxfp8.quantize(x, colwise=True)
    qtr, etr = mxfp8.quantize_ref(x.t().contiguous())
    assert qt.shape == (C, R)
    assert torch.equal(mxfp8.unchunk_scales_ref(sft, C, R), etr)
    assert torch.equal(qt.view(torch.float8_e4m3fn).float(), qtr.float())
    (q2, sf2), (qt2, sft2) = mxfp8.quantize_both(x)                 # one read, both orientations
    assert torch.equal(q2, q) and torch.equal(sf2, sf) and torch.equal(qt2, qt) and torch.equal(sft2, sft)


@pytest.mark.gpu
@pytest.mark.parametrize("M,N,K", [(128, 192, 128), (256, 384, 512), (384, 1024, 256), (200, 2048 + 64, 1024), (1024, 5632, 2048)])
def test_block_scaled_gemm_matches_dequantised_fp32(M, N, K):
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    torch.manual_seed(2)
    a = (torch.randn(M, K, device="cuda") * torch.logspace(-1, 1, K, device="cuda")).bfloat16()
    b = (torch.randn(N, K, device="cuda") * (1 + torch.arange(N, device="cuda").view(-1, 1) % 7)).bfloat16()
    aq, asf = mxfp8.quantize(a)
    bq, bsf = mxfp8.quantize(b)
    out = mxfp8.gemm(aq, asf, bq, bsf, out_f32=True)
    ar = mxfp8.dequantize_ref(aq.view(torch.float8_e4m3fn), mxfp8.unchunk_scales_ref(asf, M, K))
    br = mxfp8.dequantize_ref(bq.view(torch.float8_e4m3fn), mxfp8.unchunk_scales_ref(bsf, N, K))
    ref = ar.double() @ br.double().t()
    err = (out.double() - ref).abs().max().item()
    assert err <= 1e-4 * ref.abs().max().item(), (err, ref.abs().max().item())
    acc = torch.ones(M, N, device="cuda")
    mxfp8.gemm(aq, asf, bq, bsf, acc=acc, alpha=0.5)
    assert (acc.double() - (1 + 0.5 * ref)).abs().max().item() <= 1e-4 * ref.abs().max().item()
    from archscale_b200.ops import backend
    assert backend.require_extension().device_status() == 0


@pytest.mark.gpu
def test_linear_mxfp8_forward_backward_close_to_bf16():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    torch.manual_seed(3)
    T, K, N = 512, 256, 384
    x = torch.randn(4, T // 4, K, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(N, K, device="cuda") * 0.05).bfloat16().requires_grad_(True)
    y = mxfp8.linear_mxfp8(x, w)
    g = torch.randn_like(y)
    y.backward(g)
    xr, wr = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    yr = xr @ wr.t()
    yr.backward(g.float())
    rel = lambda a, b: ((a.float() - b).norm() / b.norm()).item()
    assert torch.allclose(y.float(), mxfp8.linear_mxfp8_ref(x.detach(), w.detach()).float(), atol=2e-2, rtol=2e-2)
    assert rel(y, yr) < 0.06 and rel(x.grad, xr.grad) < 0.06 and rel(w.grad, wr.grad) < 0.06


def test_weight_cache_keys(monkeypatch):
    """The quantised-weight cache returns the stored pair while the weight is untouched and requantises after an
    in-place change, after ``invalidate_weight_cache()`` and for the other orientation (host logic, any device)."""
    calls = []

    def fake_quantize(x, colwise=False):
        calls.append((x.data_ptr(), colwise))
        return x.clone(), torch.zeros(1)

    monkeypatch.setattr(mxfp8, "quantize", fake_quantize)
    mxfp8.invalidate_weight_cache()
    w = torch.randn(8, 8)
    a = mxfp8.quantize_weight(w, False)
    assert mxfp8.quantize_weight(w, False) is a and len(calls) == 1            # reused (checkpoint recompute, micro-steps)
    mxfp8.quantize_weight(w, True)
    assert len(calls) == 2                                                      # the other orientation is its own entry
    w.mul_(2)                                                                    # torch-visible in-place change
    assert mxfp8.quantize_weight(w, False) is not a and len(calls) == 3
    mxfp8.invalidate_weight_cache()                                              # what the optimizer step calls
    mxfp8.quantize_weight(w, False)
    assert len(calls) == 4


@pytest.mark.gpu
def test_linear_mxfp8_sees_new_weights_after_invalidation():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    torch.manual_seed(5)
    x = torch.randn(256, 256, device="cuda", dtype=torch.bfloat16)
    w = (torch.randn(128, 256, device="cuda") * 0.05).bfloat16()
    mxfp8.invalidate_weight_cache()
    y0 = mxfp8.linear_mxfp8(x, w)
    assert torch.equal(mxfp8.linear_mxfp8(x, w), y0)
    w.copy_(w * 2)
    mxfp8.invalidate_weight_cache()
    y1 = mxfp8.linear_mxfp8(x, w)
    assert ((y1.float() - 2 * y0.float()).norm() / (2 * y0.float()).norm()).item() < 0.03
