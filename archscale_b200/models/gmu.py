"""Gated Memory Unit: ``out_proj( silu(in_proj(h)) · memory )`` (or the gated-RMSNorm variant).

Reference: `lit_gpt/gated_memory_unit.py:76-126`.  ``memory`` is produced once by the SSM /
attention / MLP layer in the middle of the network and re-used by every GMU layer.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from archscale_b200 import ops
from archscale_b200.models.layers import Linear
from archscale_b200.models.norms import RMSNormGated
from archscale_b200.utils.init import torch_default_init


class GMU(nn.Module):
    def __init__(self, d_model: int, d_mem: int, bias: bool = False, use_norm: bool = False, ngroups: int = 1,
                 device=None, dtype=None) -> None:
        super().__init__()
        self.in_proj = Linear(d_model, d_mem, bias=bias, device=device, dtype=dtype)
        self.out_proj = Linear(d_mem, d_model, bias=bias, device=device, dtype=dtype)
        self.use_norm = use_norm
        if use_norm:
            self.norm = RMSNormGated(d_mem, eps=1e-5, norm_before_gate=False, group_size=d_mem // ngroups)

    def reset_parameters(self) -> None:
        for lin in (self.in_proj, self.out_proj):
            torch_default_init(lin.weight)
            if lin.bias is not None:
                nn.init.zeros_(lin.bias)
        if self.use_norm:
            self.norm.reset_parameters()

    def forward(self, hidden_states: torch.Tensor, memory: torch.Tensor) -> torch.Tensor:
        gate = self.in_proj(hidden_states)
        if self.use_norm:
            out = self.norm(memory.to(gate.dtype), gate)
        else:
            out = ops.swiglu(gate, memory.to(gate.dtype))
        return self.out_proj(out)


class GMUWrapper(nn.Module):
    def __init__(self, d_model: int, d_mem: int, bias: bool = False, use_norm: bool = False, ngroups: int = 1,
                 device=None, dtype=None) -> None:
        super().__init__()
        self.gmu = GMU(d_model, d_mem, bias, use_norm, ngroups, device, dtype)

    def reset_parameters(self) -> None:
        self.gmu.reset_parameters()

    def forward(self, hidden_states, memory):
        return self.gmu(hidden_states, memory), memory
