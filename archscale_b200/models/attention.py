"""Causal self-attention, YOCO cross-attention and differential attention modules.

Reference: `lit_gpt/attention.py:31-157` (projections, window choice, μP scale, QK-norm),
`:224-345` (forward incl. the YOCO cross branch, gate, short conv), `lit_gpt/diff_attn.py`
(head pairing, λ re-parameterisation, sub-LayerNorm).  Parameter names are the checkpoint
format: ``q_proj k_proj v_proj g_proj proj q_norm k_norm da.* attn`` (fused qkv).

The attention math itself is one call to :func:`archscale_b200.ops.attention` (tcgen05
kernel); QK-norm + RoPE is one fused call.  No host synchronisation: ``cu_seqlens`` stay on
the device and the kernel needs no ``max_seqlen``.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn

from archscale_b200 import ops
from archscale_b200.config import Config
from archscale_b200.models.layers import Linear
from archscale_b200.models.norms import FusedRMSNorm
from archscale_b200.utils.init import torch_default_init


def lambda_init_fn(depth: int) -> float:
    return 0.8 - 0.6 * math.exp(-0.3 * depth)


class DiffAttention(nn.Module):
    """Differential attention: ``softmax(q1k1ᵀ)v − λ·softmax(q2k2ᵀ)v`` on paired heads."""

    def __init__(self, head_dim: int, depth: int, softmax_scale: float, window_size=(-1, -1)) -> None:
        super().__init__()
        self.head_dim, self.depth = head_dim, depth
        self.softmax_scale, self.window_size = softmax_scale, window_size
        self.lambda_init = lambda_init_fn(depth)
        for n in ("lambda_q1", "lambda_k1", "lambda_q2", "lambda_k2"):
            setattr(self, n, nn.Parameter(torch.zeros(head_dim, dtype=torch.float32)))
        self.subln = nn.RMSNorm(2 * head_dim, eps=1e-5, elementwise_affine=True)

    def reset_parameters(self) -> None:
        self.lambda_init = lambda_init_fn(self.depth)
        for n in ("lambda_q1", "lambda_k1", "lambda_q2", "lambda_k2"):
            nn.init.normal_(getattr(self, n), mean=0.0, std=0.1)
        self.subln.reset_parameters()

    def forward(self, q, k, v, cu_seqlens=None):
        # heads are interleaved pairs: (H two) → two groups of H/2 heads
        B, T, H, D = q.shape
        G = k.shape[2]
        q1, q2 = q.view(B, T, H // 2, 2, D).unbind(3)
        k1, k2 = k.view(B, k.shape[1], G // 2, 2, D).unbind(3)
        v1, v2 = v.view(B, v.shape[1], G // 2, 2, D).unbind(3)
        kw = dict(scale=self.softmax_scale, window=self.window_size, cu_seqlens=cu_seqlens)
        # attn(q, k, [v1|v2]) as two value halves per branch keeps head_dim ≤ 128 tiles.  The four products
        # (q1,k1,v1) (q1,k1,v2) (q2,k2,v1) (q2,k2,v2) run as ONE attention call over 2·H heads (variant-major, so that every
        # variant's query heads keep their own KV heads): one launch with four times the tiles instead of four launches,
        # and three stacking copies instead of twelve strided-view copies.
        qs = torch.stack((q1, q1, q2, q2), dim=2).reshape(B, T, 2 * H, D)
        ks = torch.stack((k1, k1, k2, k2), dim=2).reshape(B, k.shape[1], 2 * G, D)
        vs = torch.stack((v1, v2, v1, v2), dim=2).reshape(B, v.shape[1], 2 * G, D)
        o = ops.attention(qs, ks, vs, **kw).view(B, T, 4, H // 2, D)
        a1 = torch.cat((o[:, :, 0], o[:, :, 1]), dim=-1)
        a2 = torch.cat((o[:, :, 2], o[:, :, 3]), dim=-1)
        lam1 = torch.exp(torch.sum(self.lambda_q1 * self.lambda_k1, dim=-1).float()).type_as(q)
        lam2 = torch.exp(torch.sum(self.lambda_q2 * self.lambda_k2, dim=-1).float()).type_as(q)
        lam = lam1 - lam2 + self.lambda_init
        a = ops.diff_combine(a1, a2, lam, self.subln.weight, 1 - self.lambda_init, 1e-5)
        # (B,T,H/2,2D) → (B,T,H,D)
        return a.reshape(B, T, H // 2, 2, D).reshape(B, T, H, D)


class CausalSelfAttention(nn.Module):
    def __init__(self, config: Config, layer_idx: int, n_embd: int, yoco_cross: bool = False) -> None:
        super().__init__()
        self.config = config
        self.yoco_cross = yoco_cross
        self.layer_idx = layer_idx
        self.local = layer_idx % config.full_per_layer < config.full_per_layer - 1
        self.head_size, self.n_head, self.n_query_groups = config.head_size, config.n_head, config.n_query_groups
        hs, H, G = self.head_size, self.n_head, self.n_query_groups
        if config.separate_qkv:
            self.q_proj = Linear(n_embd, hs * H, bias=config.attn_bias)
            if not yoco_cross:
                self.k_proj = Linear(n_embd, hs * G, bias=False)
                self.v_proj = Linear(n_embd, hs * G, bias=config.attn_bias)
            if config.gated_attn:
                self.g_proj = Linear(n_embd, H, bias=config.attn_bias)
        else:
            shape = hs * H if yoco_cross else (H + 2 * G) * hs
            if config.gated_attn:
                shape += H
            self.attn_shape = shape
            self.attn = Linear(n_embd, shape, bias=config.attn_bias)
        self.scale = config.attn_scale if config.attn_scale is not None else 1.0 / math.sqrt(hs)
        if config.mup:
            self.scale = self.scale * math.sqrt(config.mup_hd0) / math.sqrt(hs)
        if self.local and config.local_window > -1:
            self.win_tuple = (config.local_window - 1, 0)
        else:
            self.win_tuple = (-1, -1)
        self.use_cu_seqlen, self.use_da, self.qk_norm = config.use_cu_seqlen, config.use_da, config.qk_norm
        if self.qk_norm:
            self.q_norm = FusedRMSNorm(hs, eps=config.norm_eps)
            self.k_norm = FusedRMSNorm(hs, eps=config.norm_eps)
        self.use_sigmoid = config.use_sigmoid
        if self.use_sigmoid:
            # sigmoid attention with a per-head norm on its output (`lit_gpt/attention.py:77-81,353-356`)
            self.sub_norm = config.norm_class(hs, eps=config.norm_eps)
        elif self.use_da:
            depth = 10000 if config.da_const_lamb else layer_idx
            self.da = DiffAttention(hs, depth, softmax_scale=self.scale, window_size=self.win_tuple)
        if config.sink_attn:
            # learnable per-head sink logit, initialised to zero (`lit_gpt/attention.py:85-103`)
            self.softmax_offset = nn.Parameter(torch.zeros(H))
        if config.ada_rope:
            self.rope_cache = None
        if config.attn_norm:
            self.attn_norm = config.norm_class(hs * H, eps=config.norm_eps)
        self.proj = Linear(hs * H, n_embd, bias=config.attn_out_bias)
        self.sc = config.sc_attn
        self.max_len = config.block_size
        if self.sc:
            self.q_dim, self.kv_dim = H * hs, G * hs
            mk = lambda d: nn.Conv1d(d, d, kernel_size=4, groups=d, padding=3, bias=False)
            self.q_conv1d, self.k_conv1d, self.v_conv1d = mk(self.q_dim), mk(self.kv_dim), mk(self.kv_dim)
        self.z_mean = None

    def reset_parameters(self) -> None:
        for name in ("q_proj", "k_proj", "v_proj", "g_proj", "attn", "proj"):
            m = getattr(self, name, None)
            if m is not None:
                torch_default_init(m.weight)
                if m.bias is not None:
                    nn.init.zeros_(m.bias)
        for name in ("q_norm", "k_norm", "attn_norm", "sub_norm"):
            m = getattr(self, name, None)
            if m is not None and hasattr(m, "reset_parameters"):
                m.reset_parameters()
        for name in ("q_conv1d", "k_conv1d", "v_conv1d"):
            m = getattr(self, name, None)
            if m is not None:
                m.reset_parameters()
        if hasattr(self, "da"):
            self.da.reset_parameters()
        if hasattr(self, "softmax_offset"):
            nn.init.zeros_(self.softmax_offset)

    # -- rope for ada_rope layers --------------------------------------------------
    def _ada_rope(self, x: torch.Tensor, T: int):
        cfg = self.config
        if cfg.yoco_window and cfg.local_window == cfg.block_size // 2:
            initial_window, sf = 4096, cfg.scaling_factor
        else:
            initial_window, sf = cfg.local_window, 1.0
        if self.rope_cache is None or T > self.max_len:
            self.max_len = max(T, self.max_len)
            self.rope_cache = ops.build_rope_cache(self.max_len, int(cfg.rotary_percentage * cfg.head_size),
                                                   torch.bfloat16, x.device, base=0.09 * initial_window ** 1.628,
                                                   scaling_factor=sf)
        cos, sin = self.rope_cache
        return cos[:T], sin[:T]

    def _attend(self, q, k, v, cu_seqlens):
        if not self.config.fa2:
            # the reference's non-flash path: sqrt of the softmax weights over silu(v), no window / packing (`:426-441`)
            self.z_mean = None
            return ops.pointwise_attention(q, k, v, "sqrt_softmax", scale=self.scale)
        if self.use_sigmoid:
            self.z_mean = None
            out = ops.pointwise_attention(q, k, v, "sigmoid", scale=self.scale, window=self.win_tuple, cu_seqlens=cu_seqlens)
            return self.sub_norm(out)
        if self.use_da:
            self.z_mean = None
            return self.da(q, k, v, cu_seqlens=cu_seqlens)
        win = self.win_tuple
        if self.config.full_swa_extend and win == (-1, -1) and not self.training:
            win = (self.config.block_size - 1, 0)
        sink = self.softmax_offset if self.config.sink_attn else None
        want_lse = self.collect_stats
        out = ops.attention(q, k, v, scale=self.scale, window=win, cu_seqlens=cu_seqlens, sink=sink,
                            return_lse=want_lse)
        if want_lse:
            out, lse = out
            self.z_mean = (lse.float() ** 2).mean().detach()
        else:
            self.z_mean = None
        return out

    collect_stats: bool = False

    def forward(self, x: torch.Tensor, rope, max_seq_length: int, cu_seqlens: Optional[torch.Tensor] = None,
                input_pos=None, kv_cache=None, gmu_mems=None):
        B, T, C = x.shape
        cfg = self.config
        if cfg.ada_rope:
            assert cfg.local_window > 0
            rope = self._ada_rope(x, T)
        H, G, hs = self.n_head, self.n_query_groups, self.head_size
        g = None
        if self.yoco_cross:
            if cfg.separate_qkv:
                q = self.q_proj(x)
                if cfg.gated_attn:
                    g = self.g_proj(x).reshape(B, T, H, 1)
            else:
                q = self.attn(x)
                if cfg.gated_attn:
                    q, g = q.split((self.attn_shape - H, H), dim=-1)
                    g = g.reshape(B, T, H, 1)
            q = q.reshape(B, T, -1, hs)
            if not cfg.nope and not cfg.yoco_nope:
                cos, sin = rope
                q = ops.apply_rotary_emb(q, cos, sin)
            k, v = kv_cache
            y = self._attend(q, k, v, cu_seqlens)
            if cfg.gated_attn:
                y = ops.glu(g, y)
            return self.proj(y.reshape(B, T, -1)), kv_cache, gmu_mems

        fused_qkv = False
        use_rope = not cfg.nope and not (cfg.yoco_nope and self.win_tuple == (-1, -1))
        cos, sin = rope if use_rope else (None, None)
        qw = self.q_norm.weight if self.qk_norm else None
        kw = self.k_norm.weight if self.qk_norm else None

        def from_fused(y, grouped):
            """Norm + rotation read the heads in place from the projection's output and deliver dense q, k, v in one launch."""
            nonlocal fused_qkv
            if self.sc or not ops.qkv_norm_rope_supported(y, H, G, cos, qw):
                return None
            fused_qkv = True
            return ops.qkv_norm_rope(y, H, G, grouped, qw, kw, cos, sin, cfg.norm_eps)

        if cfg.separate_qkv:
            y = ops.gemm.linear_multi(x, (self.q_proj, self.k_proj, self.v_proj), keep_fused=True)
            if isinstance(y, torch.Tensor):                     # the three projections ran as one GEMM: [queries | keys | values]
                out = from_fused(y, False)
                q, k, v = out if out is not None else y.split((H * hs, G * hs, G * hs), dim=-1)
            else:
                q, k, v = y
            if cfg.gated_attn:
                g = self.g_proj(x).reshape(B, T, H, 1)
        else:
            qkv = self.attn(x)
            if cfg.gated_attn:
                qkv, g = qkv.split((self.attn_shape - H, H), dim=-1)
                g = g.reshape(B, T, H, 1)
            q_per_kv = H // G
            out = from_fused(qkv, True)                          # per group: [q_per_kv queries, key, value]
            if out is not None:
                q, k, v = out
            else:
                q, k, v = qkv.view(B, T, G, q_per_kv + 2, hs).split((q_per_kv, 1, 1), dim=-2)
        if self.sc:
            conv = lambda t, m: ops.causal_conv1d(t.reshape(B, T, -1), m.weight.squeeze(1), m.bias,
                                                  activation="silu", channel_last=True)
            q, k, v = conv(q, self.q_conv1d), conv(k, self.k_conv1d), conv(v, self.v_conv1d)
        q = q.reshape(B, T, -1, hs)
        k = k.reshape(B, T, -1, hs)
        v = v.reshape(B, T, -1, hs)
        if not fused_qkv and (self.qk_norm or use_rope):
            q, k = ops.qk_norm_rope(q, k, self.q_norm.weight if self.qk_norm else None,
                                    self.k_norm.weight if self.qk_norm else None, cos, sin, cfg.norm_eps)
        kv_cache = (k, v)
        y = self._attend(q, k, v, cu_seqlens)
        if cfg.gated_attn:
            y = ops.glu(g, y)
        y = y.reshape(B, T, -1)
        if cfg.gmu_attn:
            gmu_mems = y
        if cfg.attn_norm:
            y = self.attn_norm(y)
        return self.proj(y), kv_cache, gmu_mems
