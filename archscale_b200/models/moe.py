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
            if type(self.shared_mod_in) is Linear and self.shared_mod_in.bias is None and not self.shared_mod_in.mxfp8 \
                    and not self.shared_mod_in.nvfp4:
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
        mix = math.sqrt(0.5) if (self.share_expert and self.config.sqrt_gate) else 1.0
        mixed = False
        if self.ep_size > 1:
            from archscale_b200.parallel import ep
            routed = ep.moe_ffn_expert_parallel(h, w_in, w_out, scores, indices, self.n_mods, self.ep_group, site=id(self))
        else:
            # the shared expert's output and the 1/sqrt(2) mix are added inside the routed FFN's combine pass
            routed = ops.moe_ffn(h, w_in, w_out, scores.to(h.dtype), indices, b_in, b_out,
                                 shared=shared if self.share_expert else None, alpha=mix)
            mixed = self.share_expert
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
        if self.share_expert and not mixed:
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


class AttentionExperts(nn.Module):
    """Mixture of attention experts (`lit_gpt/moe.py:101-345` with ``is_attn=True``): every routed expert owns the q/k/v
    and output projections of ``n_head / top_k`` heads; a token's top-k experts each attend, causally and inside the
    token's own sequence, over the tokens that were routed to the same expert, and the outputs are summed with the router
    gates.  The tokens of one (expert, sequence) pair form one packed document of a variable-length attention call, RoPE
    uses the tokens' original positions with the window-derived base of the reference (`:405-417`).

    Parameters are named like the per-expert MLP variant (``router.lc_proj``, ``mods_in.weight{e}``, ``mods_out.weight{e}``).
    The expert projections run one GEMM per expert and the segment table is read on the host: this variant is never
    instantiated by the reference's own model code (`lit_gpt/model.py:443` passes ``is_attn=False``) and is kept simple."""

    def __init__(self, config: Config) -> None:
        super().__init__()
        assert not config.share_expert, "a shared expert is not supported for attention experts (`lit_gpt/moe.py:138`)"
        self.config = config
        self.aux_gamma, self.aux_style = config.aux_gamma, config.aux_style
        self.global_aux = config.global_aux and config.aux_style != "switch_seq"
        self.top_k = config.top_k
        self.n_mods = config.sparsity * config.top_k
        self.n_head = config.n_head // config.top_k
        self.n_query_groups = config.n_query_groups // config.top_k
        assert self.n_head >= 1 and self.n_query_groups >= 1 and self.n_head % self.n_query_groups == 0
        hs, C = config.head_size, config.n_embd
        self.head_size = hs
        mod_in = (self.n_head + 2 * self.n_query_groups) * hs + (self.n_head * hs if config.gated_attn else 0)
        self.mod_out_size = self.n_head * hs
        self.router = _Router(config, self.n_mods)
        self.mods_in = _PerExpertLinear(self.n_mods, C, mod_in)
        self.mods_out = _PerExpertLinear(self.n_mods, self.mod_out_size, C)
        self.scale = config.attn_scale if config.attn_scale is not None else 1.0 / math.sqrt(hs)
        if config.mup:
            self.scale = self.scale * math.sqrt(config.mup_hd0) / math.sqrt(hs)
        self.win_tuple = (config.local_window - 1, 0) if config.local_window > -1 else (-1, -1)
        self.logit_scale = config.mup_d0 / config.n_layer if (config.mup and not config.use_muon) else 1.0
        self.aux_loss = 0.0
        self.router_z_mean = None
        self.tokens_per_expert = None
        self.token_indices = None
        self.collect_stats = False
        self._rope = None

    @torch.no_grad()
    def reset_parameters(self) -> None:
        if self.config.use_muon:
            torch_default_init(self.router.lc_proj.weight)
        else:
            nn.init.normal_(self.router.lc_proj.weight, std=0.02)
        for mod in (self.mods_in, self.mods_out):
            for e in range(mod.n):
                torch_default_init(getattr(mod, f"weight{e}"))

    def _rope_cache(self, T: int, device):
        cfg = self.config
        if self._rope is None or self._rope[0].shape[0] < T or self._rope[0].device != device:
            initial_window = cfg.local_window if cfg.local_window > 0 else cfg.block_size
            self._rope = ops.build_rope_cache(max(T, cfg.block_size), int(cfg.rotary_percentage * self.head_size),
                                              torch.bfloat16, device, base=0.09 * initial_window ** 1.628,
                                              scaling_factor=cfg.scaling_factor)
        return self._rope

    @staticmethod
    def _grouped_linear(x: torch.Tensor, mod: "_PerExpertLinear", bounds) -> torch.Tensor:
        outs = []
        for e in range(mod.n):
            s, t = bounds[e], bounds[e + 1]
            w = getattr(mod, f"weight{e}")
            outs.append(ops.linear(x[s:t], w.to(x.dtype)) if t > s else x.new_zeros(0, w.shape[0]))
        return torch.cat(outs)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        B, T, C = x.shape
        h = x.reshape(-1, C)
        E, K, hs = self.n_mods, self.top_k, self.head_size
        logits = self.router.lc_proj(h).float() * self.logit_scale
        scores, indices = ops.router_topk_softmax(logits, K, self.config.sqrt_gate)
        flat = indices.reshape(-1).long()
        order = torch.argsort(flat, stable=True)                 # pairs sorted by expert, token order kept inside an expert
        tok = order // K
        counts = torch.bincount(flat, minlength=E)
        bounds = [0] + torch.cumsum(counts, 0).tolist()
        # one packed document per (expert, sequence)
        cu, _ = ops.moe.segment_cu_seqlens(tok // T, counts)
        qkv = self._grouped_linear(h[tok], self.mods_in, bounds)
        gate_dim = self.n_head * hs if self.config.gated_attn else 0
        if gate_dim:
            qkv, attn_gate = qkv.split((qkv.shape[-1] - gate_dim, gate_dim), dim=-1)
        G, qpk = self.n_query_groups, self.n_head // self.n_query_groups
        qkv = qkv.reshape(-1, G, qpk + 2, hs)
        q, k, v = qkv.split((qpk, 1, 1), dim=-2)
        q = q.reshape(1, -1, G * qpk, hs)
        k = k.reshape(1, -1, G, hs)
        v = v.reshape(1, -1, G, hs)
        if not self.config.nope:
            cos, sin = self._rope_cache(T, x.device)
            pos = (tok % T).unsqueeze(0)
            q = ops.apply_rotary_emb(q, cos, sin, False, positions=pos)
            k = ops.apply_rotary_emb(k, cos, sin, False, positions=pos)
        y = ops.attention(q.contiguous(), k.contiguous(), v.contiguous(), scale=self.scale, window=self.win_tuple, cu_seqlens=cu)
        y = y.reshape(-1, self.mod_out_size)
        if gate_dim:
            y = ops.glu(attn_gate.contiguous(), y)
        out_rows = self._grouped_linear(y, self.mods_out, bounds)
        gate = scores.reshape(-1)[order].unsqueeze(-1)
        out = torch.zeros(B * T, C, dtype=torch.float32, device=x.device)
        out.index_add_(0, tok, out_rows.float() * gate.float())
        with torch.no_grad():
            tpe = counts.to(torch.float32)
            if self.collect_stats:
                self.router_z_mean = (torch.logsumexp(logits, dim=-1) ** 2).mean()
            if self.global_aux and torch.distributed.is_available() and torch.distributed.is_initialized():
                torch.distributed.all_reduce(tpe)
            self.tokens_per_expert = tpe
            self.token_indices = indices
        if self.aux_gamma > 0:
            t_aux = tpe if self.aux_style != "switch_seq" else ops.moe.compute_tokens_per_expert_seq(indices, E, T)
            self.aux_loss = ops.load_balance_loss(F.softmax(logits, dim=-1, dtype=torch.float32), t_aux, gamma=self.aux_gamma,
                                                  global_stats=self.global_aux, style=self.aux_style, seq_len=T)
        else:
            self.aux_loss = 0.0
        return out.to(x.dtype).view(B, T, C)


def get_moe(config: Config, is_attn: bool = False, is_mlp: bool = True):
    if is_attn:
        return AttentionExperts(config)
    return SonicMoE(config, is_attn, is_mlp) if config.use_sonicmoe else MoE(config, is_attn, is_mlp)
