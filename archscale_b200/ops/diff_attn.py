"""Differential-attention combine: ``RMSNorm(a1 − λ·a2)·w·(1 − λ_init)``.

Behavioural reference: `lit_gpt/diff_attn.py:168-175` (λ re-parametrisation result applied to the two attention branches,
sub-layer RMSNorm over ``2·head_dim``, constant ``1 − λ_init`` gain).  CUDA path: ``csrc/diff_attn.cu`` — one launch
forward, one backward (dλ and the norm-gain gradient are reduced in the same kernel).
"""
from __future__ import annotations

import torch

from . import backend


def diff_combine_ref(a1, a2, lam, weight, c: float, eps: float = 1e-5):
    a = a1.float() - lam.float() * a2.float()
    a = a * torch.rsqrt(a.pow(2).mean(-1, keepdim=True) + eps) * weight.float()
    return (a * c).to(a1.dtype)


class _DiffCombineFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a1, a2, lam, weight, c, eps):
        ext = backend.require_extension()
        W = a1.shape[-1]
        x1, x2 = a1.reshape(-1, W).contiguous(), a2.reshape(-1, W).contiguous()
        lf, wf = lam.float().reshape(1).contiguous(), weight.float().contiguous()
        y, rstd = ext.diff_combine_fwd(x1, x2, lf, wf, c, eps)
        backend.count_launch()
        ctx.save_for_backward(x1, x2, lf, wf, rstd)
        ctx.meta = (c, a1.shape, lam.dtype, lam.shape, weight.dtype)
        return y.view(a1.shape)

    @staticmethod
    def backward(ctx, dy):
        ext = backend.require_extension()
        x1, x2, lf, wf, rstd = ctx.saved_tensors
        c, shape, ldt, lshape, wdt = ctx.meta
        da1, da2, dlam, dw = ext.diff_combine_bwd(dy.reshape(x1.shape).contiguous(), x1, x2, lf, wf, c, rstd)
        backend.count_launch()
        return da1.view(shape), da2.view(shape), dlam.to(ldt).view(lshape), dw.to(wdt), None, None


def diff_combine(a1, a2, lam, weight, c: float, eps: float = 1e-5):
    """a1, a2: (..., W) with W = 2·head_dim; lam: scalar tensor; weight: (W,)."""
    if (a1.is_cuda and a1.dtype == torch.bfloat16 and a2.dtype == torch.bfloat16 and a1.shape[-1] in (128, 256)
            and lam.numel() == 1 and backend.has("diff_combine_fwd") and backend.use_cuda_kernel("diff_combine", a1, a2)):
        return _DiffCombineFn.apply(a1, a2, lam, weight, float(c), eps)
    return diff_combine_ref(a1, a2, lam, weight, c, eps)
