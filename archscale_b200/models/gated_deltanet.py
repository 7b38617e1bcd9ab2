"""Gated DeltaNet mixer.

Reference: `lit_gpt/gated_deltanet.py:38-195` (projections ``q k v a b g o``, short convs,
``A_log``/``dt_bias`` init) and `:238-345` (forward: conv+SiLU → L2-normalised delta rule with
``g = −exp(A_log)·softplus(a + dt_bias)``, ``β = σ(b)·(2 if allow_neg_eigval)`` → gated RMSNorm
→ ``o_proj``; the pre-norm output is the GMU memory when ``gmu_save``).
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


class ShortConvolution(nn.Conv1d):
    """Depthwise causal conv (+SiLU) over (B,T,D) with ``cu_seqlens`` boundaries."""

    def __init__(self, hidden_size: int, kernel_size: int, bias: bool = False, activation: Optional[str] = "silu"):
        super().__init__(hidden_size, hidden_size, kernel_size, groups=hidden_size, padding=kernel_size - 1, bias=bias)
        self.activation = activation

    def forward(self, x: torch.Tensor, seq_idx: Optional[torch.Tensor] = None) -> torch.Tensor:
        return ops.causal_conv1d(x, self.weight.squeeze(1), self.bias, seq_idx=seq_idx, activation=self.activation,
                                 channel_last=True)


def seq_idx_from_cu_seqlens(cu_seqlens: torch.Tensor, total: int) -> torch.Tensor:
    pos = torch.arange(total, device=cu_seqlens.device)
    return torch.bucketize(pos, cu_seqlens[1:].to(pos.dtype), right=True).to(torch.int32).unsqueeze(0)


class GatedDeltaNet(nn.Module):
    def __init__(self, hidden_size: int = 2048, expand_v: float = 2, head_dim: int = 256, num_heads: int = 6,
                 num_v_heads: Optional[int] = None, mode: str = "chunk", use_gate: bool = True,
                 use_short_conv: bool = True, allow_neg_eigval: bool = False, conv_size: int = 4,
                 conv_bias: bool = False, layer_idx: Optional[int] = None, norm_eps: float = 1e-5,
                 gmu_save: bool = False, **_unused):
        super().__init__()
        self.mode, self.allow_neg_eigval, self.hidden_size, self.expand_v = mode, allow_neg_eigval, hidden_size, expand_v
        self.use_gate, self.use_short_conv = use_gate, use_short_conv
        self.head_dim, self.num_heads = head_dim, num_heads
        self.num_v_heads = num_v_heads if num_v_heads is not None else num_heads
        self.head_k_dim, self.head_v_dim = head_dim, int(head_dim * expand_v)
        self.key_dim, self.value_dim = num_heads * head_dim, self.num_v_heads * self.head_v_dim
        self.layer_idx, self.gmu_save = layer_idx, gmu_save
        self.q_proj = Linear(hidden_size, self.key_dim, bias=False)
        self.k_proj = Linear(hidden_size, self.key_dim, bias=False)
        self.v_proj = Linear(hidden_size, self.value_dim, bias=False)
        self.a_proj = Linear(hidden_size, self.num_v_heads, bias=False)
        self.b_proj = Linear(hidden_size, self.num_v_heads, bias=False)
        self.A_log = nn.Parameter(torch.empty(self.num_v_heads, dtype=torch.float32))
        self.dt_min, self.dt_max, self.dt_init_floor = 0.001, 0.1, 1e-4
        self.dt_bias = nn.Parameter(torch.empty(self.num_v_heads))
        if use_short_conv:
            self.q_conv1d = ShortConvolution(self.key_dim, conv_size, conv_bias, "silu")
            self.k_conv1d = ShortConvolution(self.key_dim, conv_size, conv_bias, "silu")
            self.v_conv1d = ShortConvolution(self.value_dim, conv_size, conv_bias, "silu")
        if use_gate:
            self.g_proj = Linear(hidden_size, self.value_dim, bias=False)
        self.norm = RMSNormGated(self.value_dim, eps=norm_eps, norm_before_gate=False)
        self.o_proj = Linear(self.value_dim, hidden_size, bias=False)

    @torch.no_grad()
    def reset_parameters(self) -> None:
        projs = [self.q_proj, self.k_proj, self.v_proj, self.a_proj, self.b_proj, self.o_proj]
        if self.use_gate:
            projs.append(self.g_proj)
        for p in projs:
            torch_default_init(p.weight)
        if self.use_short_conv:
            for c in (self.q_conv1d, self.k_conv1d, self.v_conv1d):
                c.reset_parameters()
        A = torch.empty(self.num_v_heads, dtype=torch.float32, device=self.A_log.device).uniform_(0, 16)
        self.A_log.copy_(torch.log(A))
        dt = torch.exp(torch.rand(self.num_v_heads, device=self.dt_bias.device, dtype=torch.float32)
                       * (math.log(self.dt_max) - math.log(self.dt_min)) + math.log(self.dt_min)
                       ).clamp(min=self.dt_init_floor)
        self.dt_bias.copy_((dt + torch.log(-torch.expm1(-dt))).to(self.dt_bias.dtype))
        self.norm.reset_parameters()

    def forward(self, hidden_states: torch.Tensor, attention_mask=None, cu_seqlens=None, gmu_mems=None):
        B, T, _ = hidden_states.shape
        q, k, v = self.q_proj(hidden_states), self.k_proj(hidden_states), self.v_proj(hidden_states)
        if self.use_short_conv:
            sidx = seq_idx_from_cu_seqlens(cu_seqlens, T) if cu_seqlens is not None else None
            q, k, v = self.q_conv1d(q, sidx), self.k_conv1d(k, sidx), self.v_conv1d(v, sidx)
        else:
            q, k, v = F.silu(q), F.silu(k), F.silu(v)
        q = q.reshape(B, T, self.num_heads, self.head_k_dim)
        k = k.reshape(B, T, self.num_heads, self.head_k_dim)
        v = v.reshape(B, T, self.num_v_heads, self.head_v_dim)
        if self.num_v_heads > self.num_heads:
            rep = self.num_v_heads // self.num_heads
            q, k = q.repeat_interleave(rep, dim=2), k.repeat_interleave(rep, dim=2)
        beta = self.b_proj(hidden_states).sigmoid()
        if self.allow_neg_eigval:
            beta = beta * 2.0
        g = -self.A_log.float().exp() * F.softplus(self.a_proj(hidden_states).float() + self.dt_bias.float())
        if attention_mask is not None:
            # padded positions neither write to nor decay the state
            m = attention_mask.to(beta.dtype).unsqueeze(-1)
            beta, g = beta * m, g * m.float()
        o = ops.gated_delta_rule(q, k, v, g, beta, l2norm=True, cu_seqlens=cu_seqlens)
        o = o.reshape(B, T, self.value_dim)
        gate = None
        if self.use_gate:
            gate = self.g_proj(hidden_states)
            if self.gmu_save:
                gmu_mems = o
        o = self.norm(o, gate)
        return self.o_proj(o), gmu_mems
