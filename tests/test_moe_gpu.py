"""MoE routing kernels and the grouped tcgen05 GEMM path vs the dense per-expert oracle."""
import pytest
import torch

from archscale_b200 import ops
from archscale_b200.ops import backend
from archscale_b200.ops.moe import moe_ffn_ref, router_topk_softmax_ref, routing_metadata_ref

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return float((a.float() - b.float()).norm() / (b.float().norm() + 1e-12))


def test_topk_indices_matches_stable_topk():
    torch.manual_seed(0)
    logits = torch.randn(4099, 64, device="cuda")
    logits[:, 5] = logits[:, 9]                 # ties: the lower index must win
    s, i = ops.router_topk_softmax(logits, 8, sqrt_gate=True)
    sr, ir = router_topk_softmax_ref(logits, 8, sqrt_gate=True)
    assert torch.equal(i, ir)
    assert torch.allclose(s, sr, atol=1e-6)


@pytest.mark.parametrize("N,E,K", [(1000, 64, 8), (37, 63, 7), (5000, 8, 2)])
def test_routing_layout_is_a_stable_aligned_sort(N, E, K):
    ext = backend.require_extension()
    torch.manual_seed(1)
    idx = torch.stack([torch.randperm(E, device="cuda")[:K] for _ in range(N)]).to(torch.int32)
    if E == 63:
        idx[idx == 17] = 18                     # an expert that receives nothing
    counts, offsets, slot_pair, pair_slot = ext.routing_layout(idx.reshape(-1).contiguous(), E)
    c_ref, _, order = routing_metadata_ref(idx, E)
    assert torch.equal(counts, c_ref)
    off = offsets.tolist()
    assert all(o % 256 == 0 for o in off) and off[0] == 0
    pos = 0
    sp = slot_pair.tolist()
    order = order.tolist()
    for e in range(E):
        n = int(counts[e])
        assert sp[off[e]:off[e] + n] == order[pos:pos + n]          # stable order inside the expert
        assert all(v == -1 for v in sp[off[e] + n:off[e + 1]])      # padding
        pos += n
    assert torch.equal(slot_pair[pair_slot.long()].cpu(), torch.arange(N * K, dtype=torch.int32))


@pytest.mark.parametrize("N,C,E,I,K", [(512, 256, 8, 128, 2), (1000, 1024, 64, 256, 8), (300, 512, 63, 64, 7)])
def test_moe_ffn_forward_backward(N, C, E, I, K):
    torch.manual_seed(2)
    x = (torch.randn(N, C, device="cuda") * 0.5).bfloat16().requires_grad_()
    w_in = (torch.randn(E, 2 * I, C, device="cuda") * 0.05).bfloat16().requires_grad_()
    w_out = (torch.randn(E, C, I, device="cuda") * 0.05).bfloat16().requires_grad_()
    logits = torch.randn(N, E, device="cuda", requires_grad=True)
    scores, idx = ops.router_topk_softmax(logits, K, sqrt_gate=True)
    out = ops.moe_ffn(x, w_in, w_out, scores, idx)
    g = torch.randn_like(out)
    out.backward(g)
    torch.cuda.synchronize()
    assert backend.require_extension().device_status() == 0
    xr, wir, wor, lr = (t.detach().float().requires_grad_() for t in (x, w_in, w_out, logits))
    sr, ir = router_topk_softmax_ref(lr, K, sqrt_gate=True)
    ref = moe_ffn_ref(xr, wir, wor, sr, ir)
    ref.backward(g.float())
    assert _rel(out, ref) < 2e-2
    assert _rel(x.grad, xr.grad) < 3e-2
    assert _rel(w_in.grad, wir.grad) < 3e-2
    assert _rel(w_out.grad, wor.grad) < 3e-2
    assert _rel(logits.grad, lr.grad) < 3e-2


def test_moe_ffn_with_shared_output_and_mix_in_the_combine_pass():
    """alpha * (routed + shared) from the combine kernel, and its gradients, against the same sum in fp32."""
    torch.manual_seed(5)
    N, C, E, I, K, alpha = 700, 512, 16, 128, 4, 0.5 ** 0.5
    x = (torch.randn(N, C, device="cuda") * 0.5).bfloat16().requires_grad_()
    w_in = (torch.randn(E, 2 * I, C, device="cuda") * 0.05).bfloat16().requires_grad_()
    w_out = (torch.randn(E, C, I, device="cuda") * 0.05).bfloat16().requires_grad_()
    shared = (torch.randn(N, C, device="cuda") * 0.3).bfloat16().requires_grad_()
    logits = torch.randn(N, E, device="cuda", requires_grad=True)
    scores, idx = ops.router_topk_softmax(logits, K, sqrt_gate=True)
    out = ops.moe_ffn(x, w_in, w_out, scores, idx, shared=shared, alpha=alpha)
    g = torch.randn_like(out)
    out.backward(g)
    torch.cuda.synchronize()
    assert backend.require_extension().device_status() == 0
    xr, wir, wor, lr, shr = (t.detach().float().requires_grad_() for t in (x, w_in, w_out, logits, shared))
    sr, ir = router_topk_softmax_ref(lr, K, sqrt_gate=True)
    ref = alpha * (moe_ffn_ref(xr, wir, wor, sr, ir) + shr)
    ref.backward(g.float())
    assert _rel(out, ref) < 2e-2
    for got, want in ((x.grad, xr.grad), (w_in.grad, wir.grad), (w_out.grad, wor.grad), (logits.grad, lr.grad),
                      (shared.grad, shr.grad)):
        assert _rel(got, want) < 3e-2


def test_grouped_gemm_with_swiglu_epilogue_equals_unfused():
    """Expert up-projection with SwiGLU in the epilogue against the grouped GEMM followed by the SwiGLU kernel."""
    ext = backend.require_extension()
    torch.manual_seed(5)
    N, C, E, I, K = 1536, 512, 8, 384, 2
    x = (torch.randn(N, C, device="cuda") * 0.5).bfloat16()
    w_in = (torch.randn(E, 2 * I, C, device="cuda") * 0.05).bfloat16()
    idx = torch.stack([torch.randperm(E, device="cuda")[:K] for _ in range(N)]).to(torch.int32)
    counts, offsets, slot_pair, pair_slot = ext.routing_layout(idx.reshape(-1).contiguous(), E)
    xs = ext.gather_rows(x, slot_pair, None, K, offsets)
    assert xs.shape[0] % 256 == 0
    h_ref = ext.grouped_gemm_bf16(0, xs, w_in.reshape(E * 2 * I, C), offsets, 0, 2 * I, C, None)
    a_ref = ext.swiglu_packed_fwd(h_ref)
    h, a = ext.grouped_gemm_swiglu(xs, w_in.reshape(E * 2 * I, C), offsets, I, True)
    rows = int(offsets[-1].item())
    assert torch.equal(h[:rows], h_ref[:rows])
    assert torch.equal(a[:rows], a_ref[:rows])
    assert ext.device_status() == 0


def test_attention_experts_gpu_matches_cpu(monkeypatch):
    """The mixture of attention experts on the GPU (bf16, variable-length attention kernel, GEMM kernels) against the
    same module in fp32 on the CPU, with the routing decision fixed (a token that flips experts under bf16 logits changes
    the attention context of every token behind it in both experts, which is not what this test is about)."""
    from archscale_b200.config import Config
    from archscale_b200.models import moe as moe_mod
    torch.manual_seed(4)
    cfg = Config(n_layer=2, n_embd=512, n_head=8, n_query_groups=4, head_dim=128, block_size=256, vocab_size=128,
                 padded_vocab_size=128, intermediate_size=1024, sparsity=2, top_k=2, sqrt_gate=True, aux_gamma=0.0)
    m = moe_mod.get_moe(cfg, is_attn=True)
    m.reset_parameters()
    x = torch.randn(2, 256, 512) * 0.5
    with torch.no_grad():
        scores, idx = router_topk_softmax_ref(m.router.lc_proj(x.reshape(-1, 512)).float(), 2, sqrt_gate=True)
    monkeypatch.setattr(moe_mod.ops, "router_topk_softmax", lambda logits, k, sq: (scores.to(logits.device), idx.to(logits.device)))
    ref = m(x)
    mg = moe_mod.get_moe(cfg, is_attn=True).cuda().bfloat16()
    mg.load_state_dict(m.state_dict())
    xg = x.cuda().bfloat16().requires_grad_()
    out = mg(xg)
    assert _rel(out.float().cpu(), ref) < 3e-2
    out.float().pow(2).mean().backward()
    assert xg.grad is not None and torch.isfinite(xg.grad).all()
