"""tcgen05 attention kernels vs the dense fp32 softmax oracle."""
import math

import pytest
import torch

from archscale_b200.ops import backend
from archscale_b200.ops.attention import attention_ref, row_start_from_cu_seqlens

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return float((a.float() - b.float()).norm() / (b.float().norm() + 1e-12))


CASES = [
    # B, T, H, G, D, window_left, cu_seqlens
    (2, 256, 4, 2, 128, -1, None),
    (1, 300, 2, 1, 128, -1, None),          # ragged tail tile
    (2, 512, 4, 4, 64, -1, None),
    (1, 640, 4, 2, 128, 99, None),          # sliding window 100
    (1, 1024, 2, 2, 64, 511, None),         # window 512, head_dim 64 (phi4-mini-flash shape)
    (1, 700, 4, 2, 128, -1, [0, 130, 131, 400, 700]),   # packed documents
    (1, 900, 2, 1, 64, 63, [0, 500, 900]),  # packed + window
    (2, 2048, 4, 2, 128, -1, None),         # many key tiles per query-tile pair
    (1, 1100, 2, 1, 128, 300, [0, 70, 610, 1100]),   # packed + window across tile pairs, odd number of query tiles
    (1, 128, 2, 2, 128, -1, None),          # a single query tile: the second CTA of the pair has no rows
]


@pytest.mark.parametrize("B,T,H,G,D,win,cu", CASES)
def test_attention_forward(B, T, H, G, D, win, cu):
    ext = backend.require_extension()
    torch.manual_seed(0)
    q = torch.randn(B, T, H, D, device="cuda").bfloat16()
    k = torch.randn(B, T, G, D, device="cuda").bfloat16()
    v = torch.randn(B, T, G, D, device="cuda").bfloat16()
    scale = 1.0 / math.sqrt(D)
    cu_t = torch.tensor(cu, device="cuda", dtype=torch.int32) if cu else None
    rs = row_start_from_cu_seqlens(cu_t, T) if cu else None
    out, lse = ext.attn_fwd_only(q, k, v, scale, win, rs)
    torch.cuda.synchronize()
    assert ext.device_status() == 0
    ref, lse_ref = attention_ref(q, k, v, scale, (win, 0) if win >= 0 else (-1, -1), cu_t, None, True)
    assert _rel(out, ref) < 2e-2, _rel(out, ref)
    assert float((lse - lse_ref).abs().max()) < 2e-2


@pytest.mark.parametrize("B,T,H,G,D,win,cu", CASES)
def test_attention_backward(B, T, H, G, D, win, cu):
    from archscale_b200 import ops
    ext = backend.require_extension()
    torch.manual_seed(1)
    q = torch.randn(B, T, H, D, device="cuda").bfloat16().requires_grad_()
    k = torch.randn(B, T, G, D, device="cuda").bfloat16().requires_grad_()
    v = torch.randn(B, T, G, D, device="cuda").bfloat16().requires_grad_()
    scale = 1.0 / math.sqrt(D)
    cu_t = torch.tensor(cu, device="cuda", dtype=torch.int32) if cu else None
    window = (win, 0) if win >= 0 else (-1, -1)
    out = ops.attention(q, k, v, scale=scale, window=window, cu_seqlens=cu_t)
    g = torch.randn_like(out)
    out.backward(g)
    torch.cuda.synchronize()
    assert ext.device_status() == 0
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    ref = attention_ref(qr, kr, vr, scale, window, cu_t)
    ref.backward(g.float())
    assert _rel(out, ref) < 2e-2
    assert _rel(q.grad, qr.grad) < 3e-2, _rel(q.grad, qr.grad)
    assert _rel(k.grad, kr.grad) < 3e-2, _rel(k.grad, kr.grad)
    assert _rel(v.grad, vr.grad) < 3e-2, _rel(v.grad, vr.grad)


def test_attention_backward_is_deterministic():
    from archscale_b200 import ops
    torch.manual_seed(2)
    q = torch.randn(2, 512, 8, 128, device="cuda").bfloat16().requires_grad_()
    k = torch.randn(2, 512, 2, 128, device="cuda").bfloat16().requires_grad_()
    v = torch.randn(2, 512, 2, 128, device="cuda").bfloat16().requires_grad_()
    g = torch.randn(2, 512, 8, 128, device="cuda").bfloat16()
    grads = []
    for _ in range(2):
        out = ops.attention(q, k, v)
        grads.append(torch.autograd.grad(out, (q, k, v), g))
    for a, b in zip(*grads):
        assert torch.equal(a, b)


@pytest.mark.parametrize("B,T,H,G,D,win,cu", [(2, 384, 4, 2, 128, -1, None), (1, 640, 4, 4, 64, 127, None),
                                               (1, 700, 4, 2, 128, -1, [0, 130, 400, 700])])
def test_sink_attention_matches_dense_softmax_with_sink_column(B, T, H, G, D, win, cu):
    """Learnable per-head sink logit on the kernel path: forward, dq/dk/dv and the sink gradient."""
    from archscale_b200 import ops
    torch.manual_seed(5)
    q = torch.randn(B, T, H, D, device="cuda").bfloat16().requires_grad_()
    k = torch.randn(B, T, G, D, device="cuda").bfloat16().requires_grad_()
    v = torch.randn(B, T, G, D, device="cuda").bfloat16().requires_grad_()
    sink = (torch.randn(H, device="cuda") * 2).requires_grad_()
    g = torch.randn(B, T, H, D, device="cuda").bfloat16()
    cu_t = torch.tensor(cu, device="cuda", dtype=torch.int32) if cu else None
    n0 = backend.launches()
    out = ops.attention(q, k, v, window=(win, 0 if win >= 0 else -1), cu_seqlens=cu_t, sink=sink)
    assert backend.launches() > n0, "sink attention did not take the kernel path"
    grads = torch.autograd.grad(out, (q, k, v, sink), g)
    assert backend.require_extension().device_status() == 0
    leaves = [t.detach().float().requires_grad_() for t in (q, k, v, sink)]
    ref = attention_ref(leaves[0], leaves[1], leaves[2], None, (win, 0 if win >= 0 else -1), cu_t, leaves[3])
    g_ref = torch.autograd.grad(ref, leaves, g.float())
    assert _rel(out, ref) < 2e-2, _rel(out, ref)
    for name, x, y in zip(("dq", "dk", "dv", "dsink"), grads, g_ref):
        assert _rel(x, y) < 3e-2, (name, _rel(x, y))
