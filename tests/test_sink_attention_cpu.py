"""The identities that put a learnable sink logit on the plain attention kernels, checked densely on CPU:
forward  lse' = logaddexp(lse, sink), out' = out·exp(lse − lse');
backward the standard flash backward fed with (out', lse') gives dq / dk / dv of the sink softmax, and
d sink_h = −Σ p_sink·δ with p_sink = exp(sink − lse'), δ = Σ_d dO·O'."""
import math

import torch

from archscale_b200.ops.attention import attention_ref


def test_sink_identities_match_dense_softmax_with_sink_column():
    torch.manual_seed(0)
    B, T, H, D = 2, 24, 3, 8
    q, k, v = (torch.randn(B, T, H, D, dtype=torch.float64) for _ in range(3))
    sink = torch.randn(H, dtype=torch.float64) * 2
    scale = 1.0 / math.sqrt(D)
    leaves = [t.clone().requires_grad_() for t in (q, k, v, sink)]
    ref = attention_ref(*leaves[:3], scale, (-1, -1), None, leaves[3])
    g = torch.randn_like(ref)
    dq_r, dk_r, dv_r, ds_r = torch.autograd.grad(ref, leaves, g)

    out, lse = attention_ref(q, k, v, scale, (-1, -1), None, None, return_lse=True)      # what the kernel returns
    lse_s = torch.logaddexp(lse, sink.view(1, H, 1))
    out_s = out * torch.exp(lse - lse_s).permute(0, 2, 1).unsqueeze(-1)
    assert torch.allclose(out_s.float(), ref.float(), atol=1e-5)

    # dense statement of the backward kernels: probabilities from the saved log-sum-exp, δ from dO·O
    qh, kh, vh, gh = (t.permute(0, 2, 1, 3) for t in (q, k, v, g))
    s = qh @ kh.transpose(-1, -2) * scale
    mask = torch.tril(torch.ones(T, T, dtype=torch.bool))
    p = torch.exp(s - lse_s.unsqueeze(-1)).masked_fill(~mask, 0.0)
    delta = (g * out_s).sum(-1).permute(0, 2, 1)                                           # (B,H,T)
    dp = gh @ vh.transpose(-1, -2)
    ds = p * (dp - delta.unsqueeze(-1))
    dq = (ds @ kh * scale).permute(0, 2, 1, 3)
    dk = (ds.transpose(-1, -2) @ qh * scale).permute(0, 2, 1, 3)
    dv = (p.transpose(-1, -2) @ gh).permute(0, 2, 1, 3)
    dsink = -(torch.exp(sink.view(1, H, 1) - lse_s) * delta).sum((0, 2))
    for a, b in ((dq, dq_r), (dk, dk_r), (dv, dv_r), (dsink, ds_r)):
        assert torch.allclose(a, b, atol=1e-6), float((a - b).abs().max())
