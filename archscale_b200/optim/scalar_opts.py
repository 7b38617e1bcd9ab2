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


def nadam_mu(beta1: float, step: int, momentum_decay: float = 4e-3) -> float:
    """Momentum coefficient of NAdam at ``step`` (1-based): ``beta1·(1 − 0.5·0.96^(step·momentum_decay))``."""
    return beta1 * (1.0 - 0.5 * (0.96 ** (step * momentum_decay)))


@torch.no_grad()
def nadam_update_foreach(x: List[torch.Tensor], g: Sequence[torch.Tensor], m: List[torch.Tensor], v: List[torch.Tensor],
                         lr: float, beta1: float, beta2: float, weight_decay: float, step: int, eps: float,
                         mu_product: float, momentum_decay: float = 4e-3) -> float:
    """NAdam with decoupled weight decay — the rule ``torch.optim.NAdam(decoupled_weight_decay=True)`` applies to the
    weight matrices of the reference's ``hadam`` runs (`pretrain.py:646-654`).  ``mu_product`` is the running product
    of the momentum coefficients of all earlier steps (1.0 before the first); the updated product is returned."""
    mu = nadam_mu(beta1, step, momentum_decay)
    mu_next = nadam_mu(beta1, step + 1, momentum_decay)
    mu_product = mu_product * mu
    if not x:
        return mu_product
    if weight_decay != 0.0:
        torch._foreach_mul_(x, 1 - lr * weight_decay)
    torch._foreach_lerp_(m, list(g), 1 - beta1)
    torch._foreach_mul_(v, beta2)
    torch._foreach_addcmul_(v, list(g), list(g), 1 - beta2)
    denom = torch._foreach_sqrt(v)
    torch._foreach_div_(denom, math.sqrt(1 - beta2 ** step))
    torch._foreach_add_(denom, eps)
    torch._foreach_addcdiv_(x, list(g), denom, value=-lr * (1.0 - mu) / (1.0 - mu_product))
    torch._foreach_addcdiv_(x, m, denom, value=-lr * mu_next / (1.0 - mu_product * mu_next))
    return mu_product
