"""Small helpers shared across the package (reference: lit_gpt/utils.py:22-36)."""
from __future__ import annotations

import torch


def find_multiple(n: int, k: int) -> int:
    """Smallest multiple of ``k`` that is >= ``n``."""
    assert k > 0
    return n if n % k == 0 else n + k - (n % k)


def num_parameters(module: torch.nn.Module, requires_grad: bool | None = None) -> int:
    return sum(p.numel() for p in module.parameters() if requires_grad is None or p.requires_grad == requires_grad)


def cdiv(a: int, b: int) -> int:
    return (a + b - 1) // b
