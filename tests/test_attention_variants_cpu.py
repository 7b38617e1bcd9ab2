"""Attention variants that run as PyTorch math: sigmoid attention, the reference's non-flash sqrt-softmax path, and the
mixture of attention experts — each against an independent per-row / per-segment statement."""
import math

import torch

from archscale_b200.config import Config
from archscale_b200.models.attention import CausalSelfAttention
from archscale_b200.models.moe import AttentionExperts, get_moe
from archscale_b200.ops.attention import attention_ref, pointwise_attention
from archscale_b200.ops.rope import apply_rotary_emb_ref, build_rope_cache


def test_sigmoid_attention_matches_row_loop_with_window_and_documents():
    torch.manual_seed(0)
    B, T, H, G, D = 2, 37, 4, 2, 8
    q = torch.randn(B, T, H, D, dtype=torch.float64)
    k, v = torch.randn(B, T, G, D, dtype=torch.float64), torch.randn(B, T, G, D, dtype=torch.float64)
    scale, W = 0.3, 5
    out = pointwise_attention(q, k, v, "sigmoid", scale=scale, window=(W - 1, 0), q_chunk=16)
    ref = torch.zeros_like(out)
    for b in range(B):
        for h in range(H):
            g = h // (H // G)
            for i in range(T):
                for j in range(max(0, i - W + 1), i + 1):
                    ref[b, i, h] += torch.sigmoid(scale * (q[b, i, h] @ k[b, j, g])) * v[b, j, g]
    assert torch.allclose(out, ref, atol=1e-5)
    # packed documents: keys of another document are invisible
    cu = torch.tensor([0, 10, 11, 37], dtype=torch.int32)
    out2 = pointwise_attention(q[:1], k[:1], v[:1], "sigmoid", scale=scale, cu_seqlens=cu)
    i = 20
    row = sum(torch.sigmoid(scale * (q[0, i, 0] @ k[0, j, 0])) * v[0, j, 0] for j in range(11, i + 1))
    assert torch.allclose(out2[0, i, 0], row, atol=1e-5)


def test_sqrt_softmax_attention_matches_dense_statement():
    torch.manual_seed(1)
    B, T, H, D = 2, 19, 2, 4
    q, k, v = (torch.randn(B, T, H, D, dtype=torch.float64) for _ in range(3))
    scale = 0.5
    out = pointwise_attention(q, k, v, "sqrt_softmax", scale=scale, q_chunk=7)
    qh, kh, vh = (t.permute(0, 2, 1, 3) for t in (q, k, v))
    mask = torch.triu(torch.ones(T, T, dtype=torch.float64), 1) * (-10000)
    y = torch.sqrt(torch.softmax(qh * scale @ kh.transpose(-1, -2) + mask, dim=-1) + 1e-5) @ torch.nn.functional.silu(vh)
    assert torch.allclose(out, y.permute(0, 2, 1, 3), atol=1e-5)


def _attn_cfg(**kw):
    return Config(n_layer=2, n_embd=64, n_head=4, n_query_groups=2, head_dim=16, block_size=32, vocab_size=128,
                  padded_vocab_size=128, intermediate_size=128, **kw)


def test_attention_module_runs_both_variants():
    torch.manual_seed(2)
    x = torch.randn(2, 32, 64)
    for kw in ({"use_sigmoid": True}, {"fa2": False}):
        cfg = _attn_cfg(**kw)
        m = CausalSelfAttention(cfg, 1, cfg.n_embd)
        m.reset_parameters()
        rope = build_rope_cache(32, int(cfg.rotary_percentage * cfg.head_size), torch.float32, x.device)
        y = m(x, rope, 32)
        y = y[0] if isinstance(y, tuple) else y
        assert y.shape == x.shape and torch.isfinite(y).all()
        y.sum().backward()
        assert all(p.grad is not None for p in m.parameters())
        assert ("sub_norm" in dict(m.named_modules())) == bool(kw.get("use_sigmoid"))


def test_attention_experts_match_per_segment_oracle():
    torch.manual_seed(3)
    cfg = _attn_cfg(sparsity=2, top_k=2, sqrt_gate=True, aux_gamma=0.01, gated_attn=True, local_window=-1)
    m = get_moe(cfg, is_attn=True)
    assert isinstance(m, AttentionExperts) and m.n_mods == 4 and m.n_head == 2 and m.n_query_groups == 1
    m.reset_parameters()
    B, T, C, hs = 2, 32, 64, 16
    x = torch.randn(B, T, C)
    out = m(x)
    assert out.shape == x.shape and float(m.aux_loss) > 0
    # oracle: per sequence and expert, attention over the tokens routed there, RoPE at the original positions
    h = x.reshape(-1, C)
    logits = m.router.lc_proj(h).float()
    vals, idx = torch.topk(logits, 2, dim=-1)
    gates = torch.sqrt(torch.softmax(vals, -1) + 1e-30)
    cos, sin = build_rope_cache(T, hs, torch.bfloat16, x.device, base=0.09 * cfg.block_size ** 1.628)
    ref = torch.zeros(B * T, C)
    for e in range(4):
        w_in, w_out = getattr(m.mods_in, f"weight{e}"), getattr(m.mods_out, f"weight{e}")
        for b in range(B):
            rows = [n for n in range(b * T, (b + 1) * T) if e in idx[n].tolist()]
            if not rows:
                continue
            r = torch.tensor(rows)
            z = h[r] @ w_in.t()
            z, gate_z = z[:, :-2 * hs], z[:, -2 * hs:]
            z = z.reshape(len(rows), 1, 4, hs)
            q, k, v = z[:, :, :2].reshape(1, -1, 2, hs), z[:, :, 2:3].reshape(1, -1, 1, hs), z[:, :, 3:].reshape(1, -1, 1, hs)
            pos = (r % T).unsqueeze(0)
            q, k = apply_rotary_emb_ref(q, cos, sin, False, positions=pos), apply_rotary_emb_ref(k, cos, sin, False, positions=pos)
            y = attention_ref(q, k, v, scale=m.scale).reshape(len(rows), 2 * hs)
            y = torch.sigmoid(gate_z) * y
            g = torch.stack([gates[n][idx[n].tolist().index(e)] for n in rows]).unsqueeze(-1)
            ref[r] += (y @ w_out.t()) * g
    assert torch.allclose(out.reshape(-1, C), ref, atol=2e-4, rtol=1e-3)
    out.sum().backward()
    assert all(p.grad is not None for p in m.parameters())


def test_differential_attention_one_call_equals_four_calls():
    """The four softmax products of differential attention run as one call over stacked heads; the result must be the
    four-call statement of the reference (`lit_gpt/diff_attn.py:161-175`)."""
    from archscale_b200.models.attention import DiffAttention
    from archscale_b200.ops.diff_attn import diff_combine_ref
    torch.manual_seed(5)
    B, T, H, G, D = 2, 24, 8, 4, 16
    da = DiffAttention(D, depth=3, softmax_scale=0.25, window_size=(7, 0))
    da.reset_parameters()
    q, k, v = torch.randn(B, T, H, D), torch.randn(B, T, G, D), torch.randn(B, T, G, D)
    out = da(q, k, v)
    q1, q2 = q.view(B, T, H // 2, 2, D).unbind(3)
    k1, k2 = k.view(B, T, G // 2, 2, D).unbind(3)
    v1, v2 = v.view(B, T, G // 2, 2, D).unbind(3)
    kw = dict(scale=0.25, window=(7, 0))
    a1 = torch.cat((attention_ref(q1, k1, v1, **kw), attention_ref(q1, k1, v2, **kw)), dim=-1)
    a2 = torch.cat((attention_ref(q2, k2, v1, **kw), attention_ref(q2, k2, v2, **kw)), dim=-1)
    lam = (torch.exp((da.lambda_q1 * da.lambda_k1).sum()) - torch.exp((da.lambda_q2 * da.lambda_k2).sum()) + da.lambda_init)
    ref = diff_combine_ref(a1, a2, lam, da.subln.weight, 1 - da.lambda_init, 1e-5).reshape(B, T, H, D)
    assert torch.allclose(out, ref, atol=1e-5, rtol=1e-5)


def test_segment_cu_seqlens_respects_sequence_and_expert_boundaries():
    """Inputs of the reference's `tests/test_build_segment_cu_seqlen.py:50-71`.  A boundary at every change of expert or of
    sequence id (the contract its helper states and implements, `:4-48`) gives four segments for the first input; the vector
    pinned there ([0, 2, 3, 5]) would let the token of sequence 2 attend to sequence 1 inside the second expert."""
    import torch
    from archscale_b200.ops.moe import segment_cu_seqlens
    cu, lens = segment_cu_seqlens(torch.tensor([0, 0, 1, 1, 2], dtype=torch.int32), torch.tensor([3, 2], dtype=torch.int32))
    assert cu.dtype == torch.int32 and lens.dtype == torch.int32
    assert cu.tolist() == [0, 2, 3, 4, 5] and lens.tolist() == [2, 1, 1, 1]
    cu, lens = segment_cu_seqlens(torch.empty(0, dtype=torch.int32), torch.empty(0, dtype=torch.int32))
    assert cu.tolist() == [0] and lens.numel() == 0 and cu.dtype == torch.int32 and lens.dtype == torch.int32
    # the same sequence id on both sides of an expert boundary still splits
    cu, lens = segment_cu_seqlens(torch.tensor([4, 4, 4, 4]), torch.tensor([1, 0, 3]))
    assert cu.tolist() == [0, 1, 4]
