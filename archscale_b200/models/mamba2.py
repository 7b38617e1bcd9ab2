"""Mamba-2 mixer (SSD scan with scalar per-head decay and gated RMSNorm).

Reference: `lit_gpt/mamba2.py:40-152` (shapes: one ``in_proj`` emitting ``[z | x B C | dt]``,
depthwise conv over ``x B C``, heads of 64, ``d_state`` 128, gated RMSNorm with
``norm_before_gate=False``), `:254-323` (split path).  The vestigial tensor-parallel hooks of
the reference (``process_group=None`` everywhere) are not reproduced.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from archscale_b200 import ops
from archscale_b200.models.layers import Linear
from archscale_b200.models.norms import RMSNormGated
from archscale_b200.utils.init import torch_default_init


class Mamba2(nn.Module):
    def __init__(self, d_model: int, d_state: int = 128, d_conv: int = 4, expand: float = 2, headdim: int = 64,
                 ngroups: int = 1, A_init_range=(1, 16), rmsnorm: bool = True, norm_before_gate: bool = False,
                 dt_min: float = 0.001, dt_max: float = 0.1, dt_init_floor: float = 1e-4, bias: bool = False,
                 conv_bias: bool = True, chunk_size: int = 256, layer_idx: Optional[int] = None,
                 gmu_save: bool = False, device=None, dtype=None, jamba_norm: bool = False, config=None):
        super().__init__()
        fk = {"device": device, "dtype": dtype}
        self.d_model, self.d_state, self.d_conv, self.headdim, self.ngroups = d_model, d_state, d_conv, headdim, ngroups
        self.d_inner = int(expand * d_model)
        self.d_ssm = self.d_inner
        assert self.d_ssm % headdim == 0
        self.nheads = self.d_ssm // headdim
        self.rmsnorm, self.norm_before_gate = rmsnorm, norm_before_gate
        self.dt_min, self.dt_max, self.dt_init_floor, self.A_init_range = dt_min, dt_max, dt_init_floor, A_init_range
        self.chunk_size, self.layer_idx, self.gmu_save = chunk_size, layer_idx, gmu_save
        d_in_proj = 2 * self.d_inner + 2 * ngroups * d_state + self.nheads
        self.in_proj = Linear(d_model, d_in_proj, bias=bias, **fk)
        conv_dim = self.d_ssm + 2 * ngroups * d_state
        self.conv1d = nn.Conv1d(conv_dim, conv_dim, bias=conv_bias, kernel_size=d_conv, groups=conv_dim,
                                padding=d_conv - 1, **fk)
        self.dt_bias = nn.Parameter(torch.empty(self.nheads, **fk))
        self.A_log = nn.Parameter(torch.empty(self.nheads, dtype=torch.float32, device=device))
        self.D = nn.Parameter(torch.empty(self.nheads, device=device))
        if rmsnorm:
            self.norm = RMSNormGated(self.d_ssm, eps=1e-5, norm_before_gate=norm_before_gate,
                                     group_size=self.d_ssm // ngroups)
        self.out_proj = Linear(self.d_inner, d_model, bias=bias, **fk)

    @torch.no_grad()
    def reset_parameters(self) -> None:
        for lin in (self.in_proj, self.out_proj):
            torch_default_init(lin.weight)
            if lin.bias is not None:
                nn.init.zeros_(lin.bias)
        torch_default_init(self.conv1d.weight)
        if self.conv1d.bias is not None:
            nn.init.zeros_(self.conv1d.bias)
        dt = torch.exp(torch.rand(self.nheads, device=self.dt_bias.device, dtype=torch.float32)
                       * (math.log(self.dt_max) - math.log(self.dt_min)) + math.log(self.dt_min)
                       ).clamp(min=self.dt_init_floor)
        self.dt_bias.copy_((dt + torch.log(-torch.expm1(-dt))).to(self.dt_bias.dtype))
        A = torch.empty(self.nheads, dtype=torch.float32, device=self.A_log.device).uniform_(*self.A_init_range)
        self.A_log.copy_(torch.log(A))
        nn.init.ones_(self.D)
        if self.rmsnorm:
            self.norm.reset_parameters()

    def forward(self, u: torch.Tensor, seq_idx=None, mask=None, gmu_mems=None):
        B, L, _ = u.shape
        zxbcdt = self.in_proj(u)
        gN = self.ngroups * self.d_state
        z, xBC, dt = torch.split(zxbcdt, [self.d_ssm, self.d_ssm + 2 * gN, self.nheads], dim=-1)
        xBC = ops.causal_conv1d(xBC, self.conv1d.weight.squeeze(1), self.conv1d.bias, seq_idx=seq_idx,
                                activation="silu", channel_last=True)
        x, Bm, Cm = torch.split(xBC, [self.d_ssm, gN, gN], dim=-1)
        dt = F.softplus(dt.float() + self.dt_bias.float())
        A = -torch.exp(self.A_log.float())
        y = ops.ssd_scan(x.reshape(B, L, self.nheads, self.headdim), dt, A,
                         Bm.reshape(B, L, self.ngroups, self.d_state), Cm.reshape(B, L, self.ngroups, self.d_state),
                         D=self.D.float(), seq_idx=seq_idx)
        y = y.reshape(B, L, self.d_ssm)
        if self.rmsnorm:
            if self.gmu_save:
                gmu_mems = y
            y = self.norm(y, z)
        else:
            y = y * F.silu(z)
        return self.out_proj(y), gmu_mems
