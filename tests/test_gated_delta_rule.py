"""Gated delta rule: chunk form vs the step-by-step oracle, the hand-derived backward of the chunk recurrence vs
autograd (CPU), and the tcgen05 recurrence kernel vs its PyTorch statement (GPU)."""
import importlib

import pytest
import torch

from archscale_b200.ops import backend

G = importlib.import_module("archscale_b200.ops.gated_delta_rule")


def _inputs(B, T, H, Dk, Dv, device="cpu", dtype=torch.float32):
    q, k = torch.randn(B, T, H, Dk, device=device, dtype=dtype), torch.randn(B, T, H, Dk, device=device, dtype=dtype)
    v = torch.randn(B, T, H, Dv, device=device, dtype=dtype)
    g = -torch.rand(B, T, H, device=device) * 0.3
    beta = torch.rand(B, T, H, device=device) * 2
    return q, k, v, g, beta


def test_chunk_form_matches_recurrence_cpu():
    torch.manual_seed(0)
    q, k, v, g, beta = _inputs(2, 150, 2, 32, 64)
    a = G.gated_delta_rule_recurrent_ref(q, k, v, g, beta)
    b = G.gated_delta_rule_chunk(q, k, v, g, beta)
    assert torch.allclose(a, b, atol=1e-5)
    cu = torch.tensor([0, 70, 150])
    a = G.gated_delta_rule_recurrent_ref(q[:1], k[:1], v[:1], g[:1], beta[:1], cu_seqlens=cu)
    b = G.gated_delta_rule_chunk(q[:1], k[:1], v[:1], g[:1], beta[:1], cu_seqlens=cu)
    assert torch.allclose(a, b, atol=1e-5)


def test_chunk_core_backward_matches_autograd_cpu():
    """_ChunkCoreFn runs the recurrence as two 'state passes' (forward, then reversed with the extra term) plus batched
    products; on CPU the passes run as their PyTorch statement, so this checks the derivation."""
    torch.manual_seed(0)
    BH, nC, c, Dk, Dv = 3, 4, 64, 32, 48
    mk = lambda *s: (torch.randn(*s, dtype=torch.float64) * 0.2).requires_grad_()
    ins = (mk(BH, nC, c, Dk), mk(BH, nC, c, Dv), mk(BH, nC, c, Dk), mk(BH, nC, c, Dk), mk(BH, nC, c, c),
           (torch.rand(BH, nC, dtype=torch.float64) * 0.5 + 0.5).requires_grad_())
    o1 = G._chunk_core_ref(*ins)
    do = torch.randn_like(o1)
    g1 = torch.autograd.grad(o1, ins, do)
    o2 = G._ChunkCoreFn.apply(*ins)
    g2 = torch.autograd.grad(o2, ins, do)
    assert torch.allclose(o1, o2, atol=1e-4)
    for x, y in zip(g1, g2):
        assert float((x - y).abs().max()) < 1e-5 * float(x.abs().max()) + 1e-5


def _rel(a, b):
    return float((a.float() - b.float()).norm() / (b.float().norm() + 1e-12))


@pytest.mark.gpu
@pytest.mark.parametrize("BH,nC,Dk,Dv,extra,reverse", [(2, 4, 256, 128, False, False), (3, 5, 128, 256, False, False),
                                                        (2, 4, 256, 256, True, True), (1, 3, 128, 128, True, True),
                                                        (6, 16, 256, 512, False, False), (6, 16, 256, 512, True, True)])
def test_state_kernel_matches_statement(BH, nC, Dk, Dv, extra, reverse):
    ext = backend.require_extension()
    torch.manual_seed(1)
    Tp = nC * 64
    mk = lambda d, s: (torch.randn(BH, Tp, d, device="cuda") * s).bfloat16()
    a_op, bm_op, c_add = mk(Dk, 0.06), mk(Dk, 0.06), mk(Dv, 1.0)
    e_op, f_op = (mk(Dv, 0.3), mk(Dk, 0.3)) if extra else (None, None)
    decay = torch.rand(BH, nC, device="cuda") * 0.5 + 0.5
    sp, sv = (1.0, -1.0) if reverse else (-1.0, 1.0)
    backend.require_extension().reset_device_status()
    v, x_all, x_fin = ext.gdn_state(a_op, c_add, bm_op, e_op, f_op, decay, reverse, sp, sv)
    torch.cuda.synchronize()
    assert ext.device_status() == 0
    v_r, x_r, xf_r = G._gdn_state_ref(a_op, c_add, bm_op, e_op, f_op, decay, reverse, sp, sv)
    assert _rel(v, v_r) < 1e-2, _rel(v, v_r)
    assert _rel(x_all, x_r) < 1e-2, _rel(x_all, x_r)
    assert _rel(x_fin, xf_r) < 1e-2, _rel(x_fin, xf_r)


@pytest.mark.gpu
@pytest.mark.parametrize("B,T,H,Dk,Dv", [(2, 256, 2, 128, 128), (1, 300, 3, 256, 512)])
def test_gated_delta_rule_gpu_forward_backward(B, T, H, Dk, Dv):
    torch.manual_seed(2)
    q, k, v, g, beta = _inputs(B, T, H, Dk, Dv, device="cuda", dtype=torch.bfloat16)
    leaves = [t.clone().requires_grad_() for t in (q, k, v, g, beta)]
    n0 = backend.launches()
    o = G.gated_delta_rule(*leaves)
    assert backend.launches() > n0, "the recurrence kernel did not run"
    do = torch.randn_like(o)
    grads = torch.autograd.grad(o, leaves, do)
    ref_leaves = [t.detach().double().requires_grad_() for t in leaves]
    o_ref = G.gated_delta_rule_recurrent_ref(*ref_leaves).double()
    g_ref = torch.autograd.grad(o_ref, ref_leaves, do.double())
    assert _rel(o, o_ref) < 2e-2, _rel(o, o_ref)
    for name, x, y in zip("q k v g beta".split(), grads, g_ref):
        assert _rel(x, y) < 4e-2, (name, _rel(x, y))


@pytest.mark.gpu
def test_gated_deltanet_block_runs_on_the_kernel():
    """A Gated DeltaNet mixer (head_dim 256, expand_v 2) forward + backward goes through the recurrence kernel."""
    from archscale_b200.models.gated_deltanet import GatedDeltaNet
    torch.manual_seed(4)
    with torch.device("cuda"):
        m = GatedDeltaNet(hidden_size=512, num_heads=2, head_dim=256, expand_v=2)
    m.reset_parameters()
    m = m.bfloat16()
    x = torch.randn(2, 200, 512, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    before = backend.launches()
    out, _ = m(x)
    out.float().square().mean().backward()
    assert backend.launches() - before >= 3
    assert torch.isfinite(out.float()).all() and torch.isfinite(x.grad.float()).all()
    for n, p in m.named_parameters():
        assert p.grad is not None and torch.isfinite(p.grad.float()).all(), n
    assert backend.require_extension().device_status() == 0


@pytest.mark.gpu
def test_unit_lower_inverse_kernel_matches_solve_and_autograd():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    from archscale_b200.ops.gated_delta_rule import unit_lower_inverse
    torch.manual_seed(4)
    A = (0.3 * torch.randn(37, 3, 64, 64, device="cuda")).tril(-1).requires_grad_()
    T = unit_lower_inverse(A)
    eye = torch.eye(64, device="cuda")
    Ar = A.detach().clone().requires_grad_()
    Tr = torch.linalg.solve_triangular(eye + Ar, eye.expand_as(Ar), upper=False, unitriangular=True)
    assert (T - Tr).abs().max() <= 1e-4 * Tr.abs().max()
    assert ((eye + A.detach()) @ T.detach() - eye).abs().max() < 1e-3
    g = torch.randn_like(T)
    T.backward(g)
    Tr.backward(g)
    assert (A.grad - Ar.grad.tril(-1)).norm() <= 1e-4 * Ar.grad.norm()
