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


def chunked_cross_entropy(logits, targets: torch.Tensor, chunk_size: int = 128) -> torch.Tensor:
    """Mean cross-entropy computed ``chunk_size`` positions at a time so that the fp32 softmax of a long sequence is never
    resident at once (`lit_gpt/utils.py:447-486`).  ``logits``: (B, T, V) tensor, or a list of (B, t_i, V) chunks as a
    chunked ``lm_head`` returns them; ``targets``: (B, T), ``-1`` entries are ignored."""
    import torch.nn.functional as F
    if isinstance(logits, (list, tuple)):
        if chunk_size == 0:
            logits = torch.cat(list(logits), dim=1)
        else:
            sizes = [l.size(1) for l in logits]
            parts = [F.cross_entropy(l.reshape(-1, l.size(-1)).float(), t.reshape(-1), ignore_index=-1, reduction="none")
                     for l, t in zip(logits, targets.split(sizes, dim=1))]
            flat = torch.cat(parts)
            return flat.sum() / (targets != -1).sum().clamp_min(1)
    logits = logits.reshape(-1, logits.size(-1))
    targets = targets.reshape(-1)
    if chunk_size == 0:
        return F.cross_entropy(logits.float(), targets, ignore_index=-1)
    parts = [F.cross_entropy(l.float(), t, ignore_index=-1, reduction="none")
             for l, t in zip(logits.split(chunk_size), targets.split(chunk_size))]
    return torch.cat(parts).sum() / (targets != -1).sum().clamp_min(1)
