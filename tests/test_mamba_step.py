"""Mamba-1 single-token decode against the full-sequence forward (CPU)."""
import torch

from archscale_b200.models.mamba import Mamba


def test_step_matches_full_forward():
    torch.manual_seed(0)
    m = Mamba(32)
    m.reset_parameters()
    x = torch.randn(2, 12, 32)
    full, _ = m(x)
    conv, ssm = m.allocate_inference_cache(2)
    outs = []
    for t in range(12):
        o, conv, ssm = m.step(x[:, t:t + 1], conv, ssm)
        outs.append(o)
    step = torch.cat(outs, dim=1)
    assert torch.allclose(step, full, atol=1e-4, rtol=1e-4), (step - full).abs().max()
