"""Normalisation modules selectable by ``Config._norm_class``.

Reference: `lit_gpt/config.py:162-229` (class switch, ``NoNorm``, weight-less ``RMSNormFunc`` /
``LayerNormFunc``), `lit_gpt/rmsnorm.py:1182-1215,1344-1364` (``FusedRMSNorm`` / ``RMSNorm``),
`lit_gpt/ops/layernorm_gated.py:388-436` (gated RMSNorm).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from archscale_b200 import ops


class FusedRMSNorm(nn.Module):
    def __init__(self, size: int, dim: int = -1, eps: float = 1e-5) -> None:
        super().__init__()
        self.weight = nn.Parameter(torch.ones(size))
        self.eps = eps

    def forward(self, x: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        return ops.rms_norm(x, self.weight, self.eps, out_dtype)

    def reset_parameters(self) -> None:
        nn.init.ones_(self.weight)


class RMSNorm(FusedRMSNorm):
    """Unfused name kept for checkpoints/flags; same math."""


class LayerNorm(nn.LayerNorm):
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.layer_norm(x, self.weight, self.bias, self.eps)


class NoNorm(nn.Module):
    def __init__(self, size: int, dim: int = -1, eps: float = 1e-5) -> None:
        super().__init__()
        self.weight = nn.Parameter(torch.ones(size))
        self.eps = eps

    def forward(self, x):
        return self.weight * x

    def reset_parameters(self) -> None:
        nn.init.ones_(self.weight)


class RMSNormFunc(nn.Module):
    """Weight-less RMSNorm; optional decoupled gain ``weight`` and skip gain ``weight1`` are
    parameters owned here but applied by the Block (post-norm variants)."""

    def __init__(self, size: Optional[int] = None, eps: float = 1e-5, decouple_gain: bool = False,
                 skip_gain: bool = False) -> None:
        super().__init__()
        self.eps, self.decouple_gain, self.skip_gain = eps, decouple_gain, skip_gain
        if decouple_gain:
            self.weight = nn.Parameter(torch.ones(size))
        if skip_gain:
            self.weight1 = nn.Parameter(torch.ones(size))

    def forward(self, x):
        return ops.rms_norm(x, None, self.eps)

    def reset_parameters(self) -> None:
        if self.decouple_gain:
            nn.init.ones_(self.weight)
        if self.skip_gain:
            nn.init.constant_(self.weight1, 1e-4)


class LayerNormFunc(nn.Module):
    def __init__(self, size: Optional[int] = None, eps: float = 1e-5) -> None:
        super().__init__()
        self.eps = eps

    def forward(self, x):
        return ops.layer_norm(x, None, None, self.eps)


class RMSNormGated(nn.Module):
    def __init__(self, size: int, eps: float = 1e-5, norm_before_gate: bool = True,
                 group_size: Optional[int] = None) -> None:
        super().__init__()
        self.weight = nn.Parameter(torch.ones(size))
        self.eps, self.norm_before_gate, self.group_size = eps, norm_before_gate, group_size

    def forward(self, x, z=None):
        return ops.gated_rms_norm(x, self.weight, z, self.eps, self.group_size, self.norm_before_gate)

    def reset_parameters(self) -> None:
        nn.init.ones_(self.weight)


_BY_NAME = {"FusedRMSNorm": FusedRMSNorm, "RMSNorm": RMSNorm, "LayerNorm": LayerNorm, "RMSNormFunc": RMSNormFunc,
            "LayerNormFunc": LayerNormFunc, "NoNorm": NoNorm}


def norm_class_by_name(name: str):
    return _BY_NAME[name]
