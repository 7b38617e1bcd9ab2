"""Mamba-2 SSD scan: the chunk-vectorised form against the step-by-step recurrence, values and gradients (CPU)."""
import pytest
import torch

from archscale_b200.ops.ssd import ssd_scan, ssd_scan_ref


@pytest.mark.parametrize("Bb,L,H,P,G,N,packed", [(2, 150, 4, 8, 1, 16, False), (1, 200, 6, 8, 2, 16, True),
                                                  (2, 128, 4, 16, 4, 8, False), (1, 37, 2, 4, 1, 4, True)])
def test_ssd_scan_matches_recurrence(Bb, L, H, P, G, N, packed):
    torch.manual_seed(0)
    x = torch.randn(Bb, L, H, P, requires_grad=True)
    dt = (torch.rand(Bb, L, H) * 0.5).requires_grad_()
    A = (-torch.rand(H) - 0.1).requires_grad_()
    B = torch.randn(Bb, L, G, N, requires_grad=True)
    C = torch.randn(Bb, L, G, N, requires_grad=True)
    D = torch.randn(H)
    seq_idx = None
    if packed:
        seq_idx = torch.zeros(Bb, L, dtype=torch.int32)
        for i, cut in enumerate((L // 3, L // 3 + 1, 2 * L // 3)):       # includes a one-token document
            seq_idx[:, cut:] = i + 1
    ins = (x, dt, A, B, C)
    y_ref = ssd_scan_ref(x, dt, A, B, C, D, seq_idx)
    y = ssd_scan(x, dt, A, B, C, D, seq_idx)
    assert torch.allclose(y, y_ref, atol=2e-4, rtol=1e-4)
    g = torch.randn_like(y)
    for a, b in zip(torch.autograd.grad(y_ref, ins, g), torch.autograd.grad(y, ins, g)):
        assert float((a - b).abs().max()) <= 2e-4 * float(a.abs().max()) + 1e-5
