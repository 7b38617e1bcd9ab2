"""Element-wise optimizer rules on lists of tensors: AdamW, Lion and their hyperball variants.

Behavioural reference: `lit_gpt/optim/scalar_opts.py:118-198` (AdamW with bias correction,
decoupled weight decay applied as ``X·(1−lr·wd)``), `:201-251` (Lion), `:254-377` (hyperball:
``X ← X − lr·(‖X‖/‖U‖)·U`` then rescale to the old norm).  State tensors are fp32.

The functions operate on *slices* (any 1-D or N-D views) so that the sharded optimizer can
pass the pieces of the flat master shards that belong to each parameter.
"""
from __future__ import annotations

import math
from typing import List, Sequence

import torch


@torch.no_grad()
def adamw_direction_(m: List[torch.Tensor], v: List[torch.Tensor], g: Sequence[torch.Tensor], beta1: float,
                     beta2: float, eps: float, step: int) -> List[torch.Tensor]:
    """Update the moments in place and return ``U = m̂ / (sqrt(v̂) + eps)`` (new tensors)."""
    torch._foreach_lerp_(m, list(g), 1 - beta1)
    torch._foreach_mul_(v, beta2)
    torch._foreach_addcmul_(v, list(g), list(g), 1 - beta2)
    bc1 = 1 - beta1 ** step
    bc2 = 1 - beta2 ** step
    denom = torch._foreach_sqrt(v)
    torch._foreach_div_(denom, math.sqrt(bc2))
    torch._foreach_add_(denom, eps)
    u = torch._foreach_div(m, denom)
    torch._foreach_div_(u, bc1)
    return u


@torch.no_grad()
def adamw_update_foreach(x: List[torch.Tensor], g: Sequence[torch.Tensor], m: List[torch.Tensor],
                         v: List[torch.Tensor], lr: float, beta1: float, beta2: float, weight_decay: float,
                         step: int, eps: float) -> None:
    if not x:
        return
    u = adamw_direction_(m, v, g, beta1, beta2, eps, step)
    if weight_decay != 0.0:
        torch._foreach_mul_(x, 1 - lr * weight_decay)
    torch._foreach_add_(x, u, alpha=-lr)


@torch.no_grad()
def lion_update_foreach(x: List[torch.Tensor], g: Sequence[torch.Tensor], m: List[torch.Tensor], lr: float,
                        beta1: float, beta2: float, weight_decay: float) -> None:
    if not x:
        return
    u = torch._foreach_lerp(m, list(g), 1 - beta1)
    u = [t.sign_() for t in u]
    torch._foreach_lerp_(m, list(g), 1 - beta2)
    if weight_decay != 0.0:
        torch._foreach_mul_(x, 1 - lr * weight_decay)
    torch._foreach_add_(x, u, alpha=-lr)
