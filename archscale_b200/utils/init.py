"""Weight initialisers.

``torch_default_init`` is the module-level switch the trainer flips for ``--ortho_init``,
``--diag_init`` and ``--maxfan_init`` (reference `utils.py:20-224`, `pretrain.py:226-231`).
The distributed variants of the reference initialise the *global* tensor and re-shard; here
modules are initialised before sharding (or from a seeded generator on every rank), so the
plain functions below already have global semantics.
"""
from __future__ import annotations

import math

import torch


def kaiming_uniform_default_(w: torch.Tensor) -> torch.Tensor:
    return torch.nn.init.kaiming_uniform_(w, a=math.sqrt(5))


def orthogonal_init_(w: torch.Tensor) -> torch.Tensor:
    if w.dim() < 2:
        return torch.nn.init.normal_(w, std=0.02)
    flat = w.new_empty(w.shape[0], w[0].numel(), dtype=torch.float32)
    torch.nn.init.orthogonal_(flat)
    with torch.no_grad():
        w.copy_(flat.view_as(w).to(w.dtype))
    return w


def diagonal_init_(w: torch.Tensor) -> torch.Tensor:
    with torch.no_grad():
        w.zero_()
        if w.dim() >= 2:
            n = min(w.shape[0], w[0].numel())
            w.view(w.shape[0], -1)[range(n), range(n)] = 1.0
    return w


def max_fan_normal_init_(w: torch.Tensor) -> torch.Tensor:
    if w.dim() < 2:
        return torch.nn.init.normal_(w, std=0.02)
    fan = max(w.shape[0], w[0].numel())
    return torch.nn.init.normal_(w, std=1.0 / math.sqrt(fan))


_current = kaiming_uniform_default_


def torch_default_init(w: torch.Tensor) -> torch.Tensor:
    return _current(w)


def set_default_init(kind: str) -> None:
    global _current
    _current = {"default": kaiming_uniform_default_, "ortho": orthogonal_init_, "diag": diagonal_init_,
                "maxfan": max_fan_normal_init_}[kind]
