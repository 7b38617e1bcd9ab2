"""Fine-grained mixture-of-experts MLP.

Reference: `lit_gpt/moe.py:421-662` (``SonicMoE``: bias-free router Linear, 3-D expert weights
``mods_in.weight (E, 2·I_e, C)`` / ``mods_out.weight (E, C, I_e)``, optional shared expert,
router z statistic, global aux loss, √½ mixing under SqrtGate) and `:42-87,101-366` (the
``use_sonicmoe=False`` variant with per-expert ``weight{e}`` parameters and ``router.lc_proj``).

Unlike the reference there is no device→host copy in ``forward``: token counts and routing
indices stay on the device (``tokens_per_expert`` is a device tensor; the logger pulls it
asynchronously).  With ``ep_size > 1`` the experts are sharded over the expert-parallel group
and tokens travel by the dispatch/combine path in :mod:`archscale_b200.parallel.ep`.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from archscale_b200 import ops
from archscale_b200.config import Config
from archscale_b200.models.layers import Linear
from archscale_b200.utils.init import torch_default_init


class Experts(nn.Module):
    """Holder of a stacked expert weight ``(E, out, in)`` (and optional bias ``(E, out)``)."""

    def __init__(self, num_experts: int, in_features: int, out_features: int, bias: bool = False) -> None:
        super().__init__()
        self.weight = nn.Parameter(torch.empty(num_experts, out_features, in_features))
        self.bias = nn.Parameter(torch.empty(num_experts, out_features)) if bias else None


class SonicMoE(nn.Module):
    def __init__(self, config: Config, is_attn: bool = False, is_mlp: bool = True) -> None:
        super().__init__()
        if is_attn:
            raise NotImplementedError("attention experts are not supported")
        self.config = config
        self.aux_gamma, self.aux_style = config.aux_gamma, config.aux_style
        self.global_aux = config.global_aux and config.aux_style != "switch_seq"
        self.share_expert = config.share_expert
        self.total_experts = config.total_experts
        if self.share_expert and config.router_top_k is None:
            assert config.top_k > 1, "shared expert requires top_k > 1"
        self.top_k = config.routed_top_k
        self.n_mods = config.routed_experts
        self.intermediate_size = config.expert_hidden
        self.ep_size = config.ep_size
        assert self.n_mods % self.ep_size == 0, "routed experts must divide evenly over the expert-parallel group"
        self.n_local = self.n_mods // self.ep_size
        self.ep_group = None  # set by parallel.ep.attach()
        C, I = config.n_embd, self.intermediate_size
        self.router = Linear(C, self.n_mods, bias=False)
        self.mods_in = Experts(self.n_local, C, 2 * I, bias=config.bias)
        self.mods_out = Experts(self.n_local, I, C, bias=config.bias)
        if self.share_expert:
            self.shared_mod_in = Linear(C, 2 * config.shared_hidden, bias=config.bias)
            self.shared_mod_out = Linear(config.shared_hidden, C, bias=config.bias)
        self.logit_scale = config.mup_d0 / config.n_layer if (config.mup and not config.use_muon) else 1.0
        self.aux_loss = 0.0
        self.router_z_mean = None
        self.tokens_per_expert = None
        self.token_indices = None
        self.collect_stats = False

    @torch.no_grad()
    def reset_parameters(self) -> None:
        if self.config.use_muon:
            torch_default_init(self.router.weight)
        else:
            nn.init.normal_(self.router.weight, std=0.02)
        for mod in (self.mods_in, self.mods_out):
            for e in range(mod.weight.shape[0]):
                torch_default_init(mod.weight[e])
            if mod.bias is not None:
                nn.init.zeros_(mod.bias)
        if self.share_expert:
            for lin in (self.shared_mod_in, self.shared_mod_out):
                torch_default_init(lin.weight)
                if lin.bias is not None:
                    nn.init.zeros_(lin.bias)

    def _router_logits(self, h: torch.Tensor) -> torch.Tensor:
        return self.router(h)

    def _expert_weights(self):
        return self.mods_in.weight, self.mods_out.weight, self.mods_in.bias, self.mods_out.bias

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        B, T, C = x.shape
        h = x.reshape(-1, C)
        if self.share_expert:
            act = None
            if type(self.shared_mod_in) is Linear and self.shared_mod_in.bias is None and not self.shared_mod_in.mxfp8:
                act = ops.linear_swiglu(h, self.shared_mod_in.weight)
            if act is None:
                act = ops.swiglu_packed(self.shared_mod_in(h))
            shared = self.shared_mod_out(act)
        # router in fp32 accumulate; logits kept for z-loss statistic and aux loss
        logits = self._router_logits(h).float() * self.logit_scale
        scores, indices = ops.router_topk_softmax(logits, self.top_k, self.config.sqrt_gate)
        w_in, w_out, b_in, b_out = self._expert_weights()
        if w_in.dtype != h.dtype:
            w_in, w_out = w_in.to(h.dtype), w_out.to(h.dtype)
        if self.ep_size > 1:
            from archscale_b200.parallel import ep
            routed = ep.moe_ffn_expert_parallel(h, w_in, w_out, scores, indices, self.n_mods, self.ep_group, site=id(self))
        else:
            routed = ops.moe_ffn(h, w_in, w_out, scores.to(h.dtype), indices, b_in, b_out)
        with torch.no_grad():
            counts = torch.bincount(indices.reshape(-1).long(), minlength=self.n_mods).to(torch.float32)
            if self.collect_stats:
                self.router_z_mean = (torch.logsumexp(logits, dim=-1) ** 2).mean()
            if self.global_aux and torch.distributed.is_available() and torch.distributed.is_initialized():
                torch.distributed.all_reduce(counts)
            self.tokens_per_expert = counts
            self.token_indices = indices
        if self.aux_gamma > 0:
            tpe = counts
            if self.aux_style == "switch_seq":
                tpe = ops.moe.compute_tokens_per_expert_seq(indices, self.n_mods, T)
            self.aux_loss = ops.load_balance_loss(F.softmax(logits, dim=-1, dtype=torch.float32), tpe,
                                                  gamma=self.aux_gamma, global_stats=self.global_aux,
                                                  style=self.aux_style, seq_len=T)
        else:
            self.aux_loss = 0.0
        if self.share_expert:
            if self.config.sqrt_gate:
                routed = math.sqrt(0.5) * routed + math.sqrt(0.5) * shared
            else:
                routed = routed + shared
        return routed.view(B, T, C)


class _PerExpertLinear(nn.Module):
    """Parameters named ``weight0 … weight{E-1}`` like a grouped linear of the reference's
    non-fused MoE (`lit_gpt/moe.py:146-150`)."""

    def __init__(self, n: int, in_features: int, out_features: int) -> None:
        super().__init__()
        self.n = n
        for e in range(n):
            setattr(self, f"weight{e}", nn.Parameter(torch.empty(out_features, in_features)))

    def stacked(self) -> torch.Tensor:
        return torch.stack([getattr(self, f"weight{e}") for e in range(self.n)])


class _Router(nn.Module):
    def __init__(self, config: Config, route_size: int) -> None:
        super().__init__()
        self.lc_proj = Linear(config.n_embd, route_size, bias=config.bias)


class MoE(SonicMoE):
    """``use_sonicmoe=False`` variant: identical math, per-expert parameter naming."""

    def __init__(self, config: Config, is_attn: bool = False, is_mlp: bool = True) -> None:
        super().__init__(config, is_attn, is_mlp)
        C, I = config.n_embd, self.intermediate_size
        del self.router, self.mods_in, self.mods_out
        self.router = _Router(config, self.n_mods)
        self.mods_in = _PerExpertLinear(self.n_local, C, 2 * I)
        self.mods_out = _PerExpertLinear(self.n_local, I, C)

    @torch.no_grad()
    def reset_parameters(self) -> None:
        if self.config.use_muon:
            torch_default_init(self.router.lc_proj.weight)
        else:
            nn.init.normal_(self.router.lc_proj.weight, std=0.02)
        for mod in (self.mods_in, self.mods_out):
            for e in range(mod.n):
                torch_default_init(getattr(mod, f"weight{e}"))
        if self.share_expert:
            for lin in (self.shared_mod_in, self.shared_mod_out):
                torch_default_init(lin.weight)

    def _router_logits(self, h: torch.Tensor) -> torch.Tensor:
        return self.router.lc_proj(h)

    def _expert_weights(self):
        return self.mods_in.stacked(), self.mods_out.stacked(), None, None


def get_moe(config: Config, is_attn: bool = False, is_mlp: bool = True):
    return SonicMoE(config, is_attn, is_mlp) if config.use_sonicmoe else MoE(config, is_attn, is_mlp)
