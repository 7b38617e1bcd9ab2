"""SSD scan on the GPU: the chunk-state recurrence kernel against its PyTorch loop, and the whole op against the recurrence."""
import pytest
import torch

from archscale_b200.ops import ssd

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("Bb,nC,H,P,N", [(2, 9, 3, 64, 16), (1, 64, 2, 64, 128), (3, 1, 1, 32, 32)])
def test_state_scan_kernel_matches_loop(Bb, nC, H, P, N):
    torch.manual_seed(1)
    add = torch.randn(Bb, nC, H, P, N, device="cuda", requires_grad=True)
    keep = torch.rand(Bb, nC, H, device="cuda").requires_grad_()
    s = ssd.chunk_state_scan(add, keep)
    assert isinstance(s.grad_fn, ssd._StateScanFn._backward_cls)          # the kernel ran, not the loop
    add_r, keep_r = add.detach().clone().requires_grad_(), keep.detach().clone().requires_grad_()
    s_r = ssd.chunk_state_scan_ref(add_r, keep_r)
    assert torch.allclose(s, s_r, atol=1e-5, rtol=1e-5)
    g = torch.randn_like(s)
    s.backward(g)
    if nC == 1:                                       # the only state is the zero initial state: nothing depends on the inputs
        assert add.grad.abs().max() == 0 and keep.grad.abs().max() == 0
        return
    s_r.backward(g)
    assert torch.allclose(add.grad, add_r.grad, atol=1e-5, rtol=1e-5)
    assert (keep.grad - keep_r.grad).abs().max() <= 1e-4 * keep_r.grad.abs().max() + 1e-5


def test_ssd_scan_gpu_matches_recurrence():
    torch.manual_seed(0)
    Bb, L, H, P, G, N = 2, 300, 4, 64, 1, 16
    x = torch.randn(Bb, L, H, P, device="cuda", requires_grad=True)
    dt = (torch.rand(Bb, L, H, device="cuda") * 0.5).requires_grad_()
    A = (-torch.rand(H, device="cuda") - 0.1).requires_grad_()
    B = torch.randn(Bb, L, G, N, device="cuda", requires_grad=True)
    C = torch.randn(Bb, L, G, N, device="cuda", requires_grad=True)
    ins = (x, dt, A, B, C)
    y_ref = ssd.ssd_scan_ref(x, dt, A, B, C)
    y = ssd.ssd_scan(x, dt, A, B, C)
    assert torch.allclose(y, y_ref, atol=2e-3, rtol=2e-3)
    g = torch.randn_like(y)
    for a, b in zip(torch.autograd.grad(y_ref, ins, g), torch.autograd.grad(y, ins, g)):
        assert float((a - b).abs().max()) <= 3e-3 * float(a.abs().max()) + 1e-4


@pytest.mark.parametrize("Bb,L,H,P,G,N,packed", [(2, 200, 4, 128, 2, 16, True), (1, 130, 6, 64, 3, 32, False)])
def test_ssd_scan_gpu_groups_wide_heads_and_documents(Bb, L, H, P, G, N, packed):
    """The intra-chunk kernel with several groups, 128-wide heads, a ragged last chunk and document breaks inside chunks."""
    torch.manual_seed(3)
    x = torch.randn(Bb, L, H, P, device="cuda", requires_grad=True)
    dt = (torch.rand(Bb, L, H, device="cuda") * 0.5).requires_grad_()
    A = (-torch.rand(H, device="cuda") - 0.1).requires_grad_()
    B = torch.randn(Bb, L, G, N, device="cuda", requires_grad=True)
    C = torch.randn(Bb, L, G, N, device="cuda", requires_grad=True)
    seq_idx = None
    if packed:
        seq_idx = torch.zeros(Bb, L, dtype=torch.int32, device="cuda")
        for i, cut in enumerate((40, 41, 150)):
            seq_idx[:, cut:] = i + 1
    ins = (x, dt, A, B, C)
    n0 = ssd.backend.launches()
    y = ssd.ssd_scan(x, dt, A, B, C, None, seq_idx)
    assert ssd.backend.launches() >= n0 + 2                  # intra-chunk kernel + state scan kernel
    y_ref = ssd.ssd_scan_ref(x, dt, A, B, C, None, seq_idx)
    assert torch.allclose(y, y_ref, atol=3e-3, rtol=3e-3)
    g = torch.randn_like(y)
    for name, a, b in zip("x dt A B C".split(), torch.autograd.grad(y_ref, ins, g), torch.autograd.grad(y, ins, g)):
        assert float((a - b).abs().max()) <= 4e-3 * float(a.abs().max()) + 1e-4, name
