"""Padding helpers, chunked cross-entropy and the activation-budget loss (CPU)."""
import torch
import torch.nn.functional as F

from archscale_b200.ops.moe import activation_budget_loss
from archscale_b200.utils.misc import chunked_cross_entropy
from archscale_b200.utils.padding import pad_input, unpad_input


def test_unpad_pad_roundtrip_and_cu_seqlens():
    torch.manual_seed(0)
    x = torch.randn(3, 7, 4, requires_grad=True)
    mask = torch.tensor([[1, 1, 1, 0, 0, 0, 0], [1, 1, 1, 1, 1, 1, 1], [1, 0, 0, 0, 0, 0, 0]], dtype=torch.bool)
    rows, idx, cu, mx = unpad_input(x, mask)
    assert rows.shape == (11, 4) and cu.tolist() == [0, 3, 10, 11] and mx == 7
    back = pad_input(rows, idx, 3, 7)
    assert torch.equal(back[mask], x[mask]) and float(back[~mask].abs().sum()) == 0.0
    back.sum().backward()
    assert torch.equal(x.grad[mask], torch.ones_like(x.grad[mask])) and float(x.grad[~mask].abs().sum()) == 0.0


def test_chunked_cross_entropy_matches_plain():
    torch.manual_seed(1)
    logits, tgt = torch.randn(2, 50, 33), torch.randint(0, 33, (2, 50))
    tgt[0, :5] = -1
    ref = F.cross_entropy(logits.reshape(-1, 33), tgt.reshape(-1), ignore_index=-1)
    assert torch.allclose(chunked_cross_entropy(logits, tgt, 16), ref, atol=1e-6)
    assert torch.allclose(chunked_cross_entropy(list(logits.split(20, dim=1)), tgt, 16), ref, atol=1e-6)
    assert torch.allclose(chunked_cross_entropy(logits, tgt, 0), ref, atol=1e-6)


def test_activation_budget_loss():
    p = torch.full((2, 3, 8), 0.25)
    assert float(activation_budget_loss(p, tau=0.25)) < 1e-12
    p2 = torch.rand(2, 3, 8)
    mask = torch.ones(2, 8)
    mask[1, 4:] = 0
    per_layer = activation_budget_loss(p2, 0.3, mask, mode="per_layer")
    frac = torch.stack([p2[0].mean(-1), p2[1, :, :4].mean(-1)])
    assert torch.allclose(per_layer, ((frac - 0.3) ** 2).mean(), atol=1e-6)
    bce = activation_budget_loss(p2, 0.3, None, loss="bce", mode="per_sequence", lambda_budget=2.0)
    m = p2.clamp(1e-6, 1 - 1e-6).mean(dim=(1, 2))
    assert torch.allclose(bce, 2.0 * F.binary_cross_entropy(m, torch.full_like(m, 0.3)), atol=1e-6)


def test_incremental_save_and_lazy_load(tmp_path):
    import torch
    from archscale_b200.utils.lazy_ckpt import incremental_save, lazy_load
    p = tmp_path / "ckpt.pth"
    a, b, c = torch.randn(5, 7), torch.arange(10, dtype=torch.bfloat16), torch.randn(4, 4)[:, 1:3]
    with incremental_save(p) as s:
        tree = {"model": {"a": s.store_early(a), "b": s.store_early(b)}, "late": c, "iter_num": 3,
                "param": torch.nn.Parameter(torch.ones(2))}
        s.save(tree)
    x = torch.load(p, weights_only=True)                 # an ordinary torch checkpoint
    assert torch.equal(x["model"]["a"], a) and torch.equal(x["model"]["b"], b) and torch.equal(x["late"], c)
    assert x["iter_num"] == 3 and torch.equal(x["param"], torch.ones(2))
    with lazy_load(p) as sd:                              # tensors mapped from the file, read on access
        assert torch.equal(sd["model"]["a"], a) and sd["model"]["b"].dtype == torch.bfloat16


def test_bench_cfg_overrides_are_typed():
    import importlib.util
    import os
    spec = importlib.util.spec_from_file_location("bench_mod", os.path.join(os.path.dirname(os.path.dirname(__file__)), "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    got = bench.parse_cfg_overrides(["residual_in_fp32=true", "n_layer=4", "norm_eps=1e-6", "aux_style=switch_seq", "qk_norm=False"])
    assert got == {"residual_in_fp32": True, "n_layer": 4, "norm_eps": 1e-6, "aux_style": "switch_seq", "qk_norm": False}
    import pytest
    with pytest.raises(ValueError):
        bench.parse_cfg_overrides(["no_equals_sign"])


def test_moe_ffn_adds_the_shared_output_and_the_mix_on_cpu():
    """``moe_ffn(..., shared, alpha)`` = alpha · (routed + shared), values and gradients, on the PyTorch path."""
    import torch
    from archscale_b200 import ops
    from archscale_b200.ops.moe import moe_ffn_ref, router_topk_softmax_ref
    torch.manual_seed(0)
    N, C, E, I, K, alpha = 40, 16, 4, 8, 2, 0.5 ** 0.5
    x = torch.randn(N, C, requires_grad=True)
    w_in = (torch.randn(E, 2 * I, C) * 0.2).requires_grad_()
    w_out = (torch.randn(E, C, I) * 0.2).requires_grad_()
    shared = torch.randn(N, C, requires_grad=True)
    scores, idx = router_topk_softmax_ref(torch.randn(N, E), K, sqrt_gate=True)
    out = ops.moe_ffn(x, w_in, w_out, scores, idx, shared=shared, alpha=alpha)
    g = torch.randn_like(out)
    out.backward(g)
    xr, wir, wor, shr = (t.detach().clone().requires_grad_() for t in (x, w_in, w_out, shared))
    ref = alpha * (moe_ffn_ref(xr, wir, wor, scores, idx) + shr)
    ref.backward(g)
    assert torch.allclose(out, ref, atol=1e-5)
    for a, b in ((x.grad, xr.grad), (w_in.grad, wir.grad), (w_out.grad, wor.grad), (shared.grad, shr.grad)):
        assert torch.allclose(a, b, atol=1e-5)


def test_guard_bands_and_run_twice_comparison():
    import torch
    from archscale_b200.utils import canary
    v, raw = canary.guarded((3, 5), torch.float32, "cpu")
    assert v.shape == (3, 5) and float(v.abs().sum()) == 0.0 and canary.guards_intact(v, raw)
    v.fill_(7.0)                                               # writes inside the tensor leave the bands alone
    assert canary.guards_intact(v, raw)
    raw[canary._GUARD_BYTES + v.numel() * 4 + 2] = 0           # one byte past the end
    assert not canary.guards_intact(v, raw)
    v2, raw2 = canary.guarded((4,), torch.bfloat16, "cpu")
    raw2[canary._GUARD_BYTES - 1] = 0                          # one byte before the start
    assert not canary.guards_intact(v2, raw2)
    x = torch.randn(8, 8)
    assert canary.bitwise_repeatable(lambda: (x @ x, None, [x + 1]))
    state = {"n": 0}

    def drifting():
        state["n"] += 1
        return x + state["n"] * 1e-7
    assert not canary.bitwise_repeatable(drifting)
