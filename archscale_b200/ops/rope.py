"""Rotary position embedding (NeoX halves or interleaved pairs) and the cos/sin cache.

Behavioural reference: `lit_gpt/fused_rotary_embedding.py:28-40,43-95` (rotation and its
conjugate backward) and `lit_gpt/attention.py:443-507` (cache with YaRN concentration and
NTK-by-parts interpolation).  Call sites use ``interleaved=False``.

CUDA path: ``csrc/rope.cu`` (fused with the per-head QK RMSNorm, see :func:`qk_norm_rope`).
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

from . import backend
from .norm import rms_norm_ref


def build_rope_cache(seq_len: int, n_elem: int, dtype: torch.dtype, device, base: float = 10000,
                     ntk_alpha: float = 1.0, ntk_beta: float = 32.0, scaling_factor: float = 1.0,
                     initial_context_length: int = 4096) -> Tuple[torch.Tensor, torch.Tensor]:
    freq = base ** (torch.arange(0, n_elem, 2, device=device) / n_elem)
    if scaling_factor > 1.0:
        concentration = 0.1 * math.log(scaling_factor) + 1.0
        d_half = n_elem / 2
        low = d_half * math.log(initial_context_length / (ntk_beta * 2 * math.pi)) / math.log(base)
        high = d_half * math.log(initial_context_length / (ntk_alpha * 2 * math.pi)) / math.log(base)
        assert 0 < low < high < d_half - 1
        ramp = (torch.arange(d_half, dtype=torch.float32, device=device) - low) / (high - low)
        keep = 1 - ramp.clamp(0, 1)  # 1 → extrapolate (high-frequency dims), 0 → interpolate
        inv_freq = (1.0 / (scaling_factor * freq)) * (1 - keep) + (1.0 / freq) * keep
    else:
        concentration = 1.0
        inv_freq = 1.0 / freq
    theta = torch.outer(torch.arange(seq_len, device=device), inv_freq)
    cos, sin = torch.cos(theta) * concentration, torch.sin(theta) * concentration
    if dtype == torch.bfloat16:
        return cos.bfloat16(), sin.bfloat16()
    if dtype in (torch.float16, torch.int8):
        return cos.half(), sin.half()
    return cos, sin


def _rotate(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, interleaved: bool, conj: bool,
            positions: Optional[torch.Tensor]) -> torch.Tensor:
    # x: (..., T, H, D); cos/sin: (T_cache, R/2) with R <= D
    T = x.shape[-3]
    if positions is not None:
        cos, sin = cos[positions], sin[positions]
    else:
        cos, sin = cos[:T], sin[:T]
    r = cos.shape[-1] * 2
    cos = cos.float().unsqueeze(-2)
    sin = sin.float().unsqueeze(-2)
    if conj:
        sin = -sin
    xr = x[..., :r].float()
    if interleaved:
        x0, x1 = xr[..., 0::2], xr[..., 1::2]
        o = torch.stack((x0 * cos - x1 * sin, x0 * sin + x1 * cos), dim=-1).flatten(-2)
    else:
        x0, x1 = xr[..., : r // 2], xr[..., r // 2:]
        o = torch.cat((x0 * cos - x1 * sin, x0 * sin + x1 * cos), dim=-1)
    return torch.cat((o.to(x.dtype), x[..., r:]), dim=-1) if r < x.shape[-1] else o.to(x.dtype)


class _RopeRef(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cos, sin, interleaved, positions):
        ctx.save_for_backward(cos, sin, positions if positions is not None else torch.empty(0))
        ctx.interleaved = interleaved
        ctx.has_pos = positions is not None
        return _rotate(x, cos, sin, interleaved, False, positions)

    @staticmethod
    def backward(ctx, do):
        cos, sin, pos = ctx.saved_tensors
        return _rotate(do, cos, sin, ctx.interleaved, True, pos if ctx.has_pos else None), None, None, None, None


def apply_rotary_emb_ref(x, cos, sin, interleaved: bool = False, positions=None):
    return _RopeRef.apply(x, cos, sin, interleaved, positions)


def qk_norm_rope_ref(q, k, q_weight, k_weight, cos, sin, eps: float = 1e-5, positions=None):
    """Per-head RMSNorm over head_dim (optional) followed by RoPE (optional) on q and k."""
    if q_weight is not None:
        q = rms_norm_ref(q, q_weight, eps)
        k = rms_norm_ref(k, k_weight, eps)
    if cos is not None:
        q = apply_rotary_emb_ref(q, cos, sin, False, positions)
        k = apply_rotary_emb_ref(k, cos, sin, False, positions)
    return q, k


def _rows_ok(t: torch.Tensor) -> torch.Tensor:
    """(B,T,H,D) with dense head rows and a uniform token stride (a column slice of a fused projection qualifies)."""
    if t.stride(3) == 1 and t.stride(2) == t.size(3) and (t.size(0) == 1 or t.stride(0) == t.size(1) * t.stride(1)):
        return t
    return t.contiguous()


class _QKNormRopeFn(torch.autograd.Function):
    """q:(B,T,H,D) k:(B,T,G,D) bf16 → normalised+rotated copies; one launch fwd, one bwd."""

    @staticmethod
    def forward(ctx, q, k, qw, kw, cos, sin, eps):
        ext = backend.require_extension()
        q, k = _rows_ok(q), _rows_ok(k)
        qo, ko, q_rstd, k_rstd = ext.qknorm_rope_fwd(q, k, qw, kw, cos, sin, eps)
        backend.count_launch()
        ctx.save_for_backward(q, k, qw, kw, cos, sin, q_rstd, k_rstd)
        return qo, ko

    @staticmethod
    def backward(ctx, dqo, dko):
        ext = backend.require_extension()
        q, k, qw, kw, cos, sin, q_rstd, k_rstd = ctx.saved_tensors
        dq, dk, dqw, dkw = ext.qknorm_rope_bwd(dqo.contiguous(), dko.contiguous(), q, k, qw, kw, cos, sin,
                                               q_rstd, k_rstd)
        backend.count_launch()
        if qw is not None:
            dqw, dkw = dqw.to(qw.dtype), dkw.to(kw.dtype)
        return dq, dk, dqw, dkw, None, None, None


def qk_norm_rope(q, k, q_weight, k_weight, cos, sin, eps: float = 1e-5, positions=None):
    D = q.shape[-1]
    full_rot = cos is None or cos.shape[-1] * 2 == D
    if (q.dim() == 4 and q.dtype == torch.bfloat16 and positions is None and full_rot and D in (64, 128)
            and (q_weight is not None or cos is not None)
            and backend.use_cuda_kernel("qknorm_rope", q, k)):
        if cos is not None:
            cos, sin = cos[: q.shape[1]].contiguous(), sin[: q.shape[1]].contiguous()
        return _QKNormRopeFn.apply(q, k, q_weight, k_weight, cos, sin, eps)
    return qk_norm_rope_ref(q, k, q_weight, k_weight, cos, sin, eps, positions)


class _QKVNormRopeFn(torch.autograd.Function):
    """The fused QKV projection output [B,T,(H+2G)·D] → (q', k', v): per-head RMSNorm + RoPE on the query and key heads read in
    place, the value heads copied to dense rows, one launch; backward writes dq, dk and dv into one tensor of the projection's
    layout (no split copies forward, no concatenation backward).  ``grouped``: per key/value group [queries, key, value] (one
    fused ``attn`` projection, the checkpoint layout of the reference); else blocked [queries | keys | values] (the q / k / v
    projections run as one GEMM)."""

    @staticmethod
    def forward(ctx, qkv, H, G, grouped, qw, kw, cos, sin, eps):
        ext = backend.require_extension()
        qo, ko, vo, q_rstd, k_rstd = ext.qkvnorm_rope_fwd(qkv, H, G, grouped, qw, kw, cos, sin, eps)
        backend.count_launch()
        ctx.save_for_backward(qkv, qw, kw, cos, sin, q_rstd, k_rstd)
        ctx.meta = (H, G, grouped)
        return qo, ko, vo

    @staticmethod
    def backward(ctx, dqo, dko, dvo):
        ext = backend.require_extension()
        qkv, qw, kw, cos, sin, q_rstd, k_rstd = ctx.saved_tensors
        H, G, grouped = ctx.meta
        B, T, W = qkv.shape
        D = W // (H + 2 * G)
        zeros = lambda heads: torch.zeros(B, T, heads, D, dtype=qkv.dtype, device=qkv.device)
        dqo = zeros(H) if dqo is None else dqo.contiguous()
        dko = zeros(G) if dko is None else dko.contiguous()
        dvo = zeros(G) if dvo is None else dvo.contiguous()
        dqkv, dqw, dkw = ext.qkvnorm_rope_bwd(dqo, dko, dvo, qkv, H, G, grouped, qw, kw, cos, sin, q_rstd, k_rstd)
        backend.count_launch()
        if qw is not None:
            dqw, dkw = dqw.to(qw.dtype), dkw.to(kw.dtype)
        else:
            dqw = dkw = None
        return dqkv, None, None, None, dqw, dkw, None, None, None


def qkv_norm_rope_supported(qkv: torch.Tensor, H: int, G: int, cos, q_weight) -> bool:
    """The fused path takes a bf16 CUDA tensor [B,T,(H+2G)·D] with a dense last dimension and a uniform token stride, D 64 or
    128, a full rotation (or none) and at least one of norm / rotation to apply."""
    if not (qkv.dim() == 3 and qkv.is_cuda and qkv.dtype == torch.bfloat16 and H % G == 0 and qkv.shape[-1] % (H + 2 * G) == 0):
        return False
    B, T, W = qkv.shape
    D = W // (H + 2 * G)
    if D not in (64, 128) or qkv.stride(2) != 1 or not (B == 1 or qkv.stride(0) == T * qkv.stride(1)):
        return False
    if cos is None and q_weight is None:
        return False
    if cos is not None and cos.shape[-1] * 2 != D:
        return False
    return backend.has("qkvnorm_rope_fwd") and backend.use_cuda_kernel("qkv_fused", qkv)


def qkv_norm_rope(qkv, H: int, G: int, grouped: bool, q_weight, k_weight, cos, sin, eps: float = 1e-5):
    """(q' [B,T,H,D], k' [B,T,G,D], v [B,T,G,D]) from the fused projection output; see :class:`_QKVNormRopeFn`.  Callers check
    :func:`qkv_norm_rope_supported` first."""
    if cos is not None:
        cos, sin = cos[: qkv.shape[1]].contiguous(), sin[: qkv.shape[1]].contiguous()
    return _QKVNormRopeFn.apply(qkv, H, G, grouped, q_weight, k_weight, cos, sin, eps)


def apply_rotary_emb(x, cos, sin, interleaved: bool = False, positions=None):
    return apply_rotary_emb_ref(x, cos, sin, interleaved, positions)
