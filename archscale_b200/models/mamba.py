"""Mamba-1 mixer (selective state space) with GMU memory export.

Reference: `lit_gpt/mamba_simple.py:36-121` (shapes), `:123-183` (init), `:248-361`
(conv1d → x_proj → dt_proj → selective scan → SwiGLU gate → out_proj; with ``gmu_save`` the
scan output *before* the ``·silu(z)`` gate is exported as the GMU memory).  Parameter names
(``in_proj x_proj dt_proj out_proj conv1d A_log D``) are the checkpoint format.

Layout: activations stay token-major ``(B, L, d_inner)`` end to end (the conv and scan
kernels are channel-last), so there are no ``b l d ↔ b d l`` transposes around the GEMMs.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from archscale_b200 import ops
from archscale_b200.models.layers import Linear
from archscale_b200.models.norms import FusedRMSNorm
from archscale_b200.utils.init import torch_default_init


class Mamba(nn.Module):
    def __init__(self, d_model: int, d_state: int = 16, d_conv: int = 4, expand: int = 2, dt_rank="auto",
                 dt_min: float = 0.001, dt_max: float = 0.1, dt_init: str = "random", dt_scale: float = 1.0,
                 dt_init_floor: float = 1e-4, jamba_norm: bool = False, conv_bias: bool = True, bias: bool = False,
                 layer_idx: Optional[int] = None, gmu_save: bool = False, config=None, device=None, dtype=None):
        super().__init__()
        fk = {"device": device, "dtype": dtype}
        self.d_model, self.d_state, self.d_conv, self.expand = d_model, d_state, d_conv, expand
        self.d_inner = int(expand * d_model)
        self.dt_rank = math.ceil(d_model / 16) if dt_rank == "auto" else dt_rank
        self.dt_min, self.dt_max, self.dt_init_floor = dt_min, dt_max, dt_init_floor
        self.dt_init, self.dt_scale = dt_init, dt_scale
        self.layer_idx, self.jamba_norm, self.gmu_save = layer_idx, jamba_norm, gmu_save
        self.use_cu_seqlen = bool(config is not None and config.use_cu_seqlen)
        if jamba_norm:
            self.dt_layernorm = FusedRMSNorm(self.dt_rank, eps=1e-5)
            self.b_layernorm = FusedRMSNorm(d_state, eps=1e-5)
            self.c_layernorm = FusedRMSNorm(d_state, eps=1e-5)
        self.in_proj = Linear(d_model, self.d_inner * 2, bias=bias, **fk)
        self.conv1d = nn.Conv1d(self.d_inner, self.d_inner, bias=conv_bias, kernel_size=d_conv, groups=self.d_inner,
                                padding=d_conv - 1, **fk)
        self.x_proj = Linear(self.d_inner, self.dt_rank + 2 * d_state, bias=False, **fk)
        self.dt_proj = Linear(self.dt_rank, self.d_inner, bias=True, **fk)
        self.A_log = nn.Parameter(torch.ones(self.d_inner, d_state, dtype=torch.float32, device=device))
        self.D = nn.Parameter(torch.ones(self.d_inner, dtype=torch.float32, device=device))
        self.out_proj = Linear(self.d_inner, d_model, bias=bias, **fk)

    @torch.no_grad()
    def reset_parameters(self) -> None:
        for lin in (self.in_proj, self.x_proj, self.out_proj):
            torch_default_init(lin.weight)
            if lin.bias is not None:
                nn.init.zeros_(lin.bias)
        torch_default_init(self.conv1d.weight)
        if self.conv1d.bias is not None:
            nn.init.zeros_(self.conv1d.bias)
        std = self.dt_rank ** -0.5 * self.dt_scale
        if self.dt_init == "constant":
            nn.init.constant_(self.dt_proj.weight, std)
        else:
            nn.init.uniform_(self.dt_proj.weight, -std, std)
        dt = torch.exp(torch.rand(self.d_inner, device=self.dt_proj.bias.device, dtype=torch.float32)
                       * (math.log(self.dt_max) - math.log(self.dt_min)) + math.log(self.dt_min)
                       ).clamp(min=self.dt_init_floor)
        self.dt_proj.bias.copy_((dt + torch.log(-torch.expm1(-dt))).to(self.dt_proj.bias.dtype))  # softplus⁻¹
        A = torch.arange(1, self.d_state + 1, dtype=torch.float32, device=self.A_log.device)
        self.A_log.copy_(torch.log(A).expand(self.d_inner, -1))
        nn.init.ones_(self.D)
        if self.jamba_norm:
            for m in (self.dt_layernorm, self.b_layernorm, self.c_layernorm):
                m.reset_parameters()

    def forward(self, hidden_states: torch.Tensor, seq_idx=None, mask=None, gmu_mems=None):
        """hidden_states:(B,L,C).  ``mask`` is ``cu_seqlens`` when the config packs documents, else an
        optional (B,L) 0/1 padding mask.  Returns (out, gmu_mems)."""
        B, L, _ = hidden_states.shape
        xz = self.in_proj(hidden_states)                       # (B,L,2·Di) token-major
        x, z = xz.split(self.d_inner, dim=-1)
        cu = mask if self.use_cu_seqlen else None
        pad_mask = mask if (mask is not None and not self.use_cu_seqlen) else None
        if pad_mask is not None:
            x = x * pad_mask.unsqueeze(-1).to(x.dtype)
        x = ops.causal_conv1d(x, self.conv1d.weight.squeeze(1), self.conv1d.bias,
                              seq_idx=seq_idx if self.use_cu_seqlen else None, activation="silu", channel_last=True)
        if pad_mask is not None:
            x = x * pad_mask.unsqueeze(-1).to(x.dtype)
        x_dbl = self.x_proj(x)                                 # (B,L,R+2N)
        dt, Bm, Cm = torch.split(x_dbl, [self.dt_rank, self.d_state, self.d_state], dim=-1)
        if self.jamba_norm:
            dt, Bm, Cm = self.dt_layernorm(dt), self.b_layernorm(Bm), self.c_layernorm(Cm)
        dt = F.linear(dt, self.dt_proj.weight.to(dt.dtype))    # bias is added inside the scan (fp32)
        A = -torch.exp(self.A_log.float())
        y = ops.selective_scan(x, dt, A, Bm, Cm, self.D.float(), z=None if self.gmu_save else z,
                               delta_bias=self.dt_proj.bias.float(), delta_softplus=True, cu_seqlens=cu, channel_last=True)
        if self.gmu_save:
            gmu_mems = y
            y = ops.swiglu(z.contiguous(), y.contiguous())
        return self.out_proj(y), gmu_mems

    # -- single-token decode (`lit_gpt/mamba_simple.py:363-408`) -----------------------------------------------------
    def allocate_inference_cache(self, batch_size: int, device=None, dtype=None):
        """(conv_state (B, d_inner, d_conv), ssm_state (B, d_inner, d_state)) filled with zeros."""
        device = device or self.out_proj.weight.device
        dtype = dtype or self.conv1d.weight.dtype
        return (torch.zeros(batch_size, self.d_inner, self.d_conv, device=device, dtype=dtype),
                torch.zeros(batch_size, self.d_inner, self.d_state, device=device, dtype=torch.float32))

    @torch.no_grad()
    def step(self, hidden_states: torch.Tensor, conv_state: torch.Tensor, ssm_state: torch.Tensor):
        """One token: hidden_states (B, 1, C); the states are updated in place and returned with the output."""
        assert hidden_states.shape[1] == 1, "step() decodes one token at a time"
        dtype = hidden_states.dtype
        xz = self.in_proj(hidden_states.squeeze(1))
        x, z = xz.chunk(2, dim=-1)
        conv_state.copy_(torch.roll(conv_state, shifts=-1, dims=-1))
        conv_state[:, :, -1] = x
        x = torch.sum(conv_state.float() * self.conv1d.weight.squeeze(1).float(), dim=-1)
        if self.conv1d.bias is not None:
            x = x + self.conv1d.bias.float()
        x = F.silu(x).to(dtype)
        dt, Bm, Cm = torch.split(self.x_proj(x), [self.dt_rank, self.d_state, self.d_state], dim=-1)
        if self.jamba_norm:
            dt, Bm, Cm = self.dt_layernorm(dt), self.b_layernorm(Bm), self.c_layernorm(Cm)
        dt = F.softplus(F.linear(dt, self.dt_proj.weight.to(dt.dtype)).float() + self.dt_proj.bias.float())
        A = -torch.exp(self.A_log.float())
        dA = torch.exp(torch.einsum("bd,dn->bdn", dt, A))
        dB = torch.einsum("bd,bn->bdn", dt, Bm.float())
        ssm_state.copy_(ssm_state * dA + x.float().unsqueeze(-1) * dB)
        y = torch.einsum("bdn,bn->bd", ssm_state, Cm.float()) + self.D.float() * x.float()
        if self.gmu_save:
            mem = y.to(dtype)
            y = y * F.silu(z.float())
            return self.out_proj(y.to(dtype)).unsqueeze(1), conv_state, ssm_state, mem.unsqueeze(1)
        y = y * F.silu(z.float())
        return self.out_proj(y.to(dtype)).unsqueeze(1), conv_state, ssm_state
