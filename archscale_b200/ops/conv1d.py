"""Depthwise causal conv1d (+SiLU) with packed-sequence boundaries.

Behavioural reference: the ``causal_conv1d_fn`` calls at `lit_gpt/mamba_simple.py:265-278`,
`lit_gpt/attention.py:300-317`: ``y[b,c,t] = act(bias[c] + Σ_j w[c,j]·x[b,c,t-(W-1)+j])`` with
zero left padding; with ``seq_idx`` taps that would reach into a different document read 0.

CUDA path: ``csrc/conv1d.cu`` (channel-last tiles, W ≤ 4 taps in registers, fwd + bwd).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F

from . import backend


def causal_conv1d_ref(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
                      seq_idx: Optional[torch.Tensor] = None, activation: Optional[str] = None) -> torch.Tensor:
    """x:(B,C,L) weight:(C,W) bias:(C,) seq_idx:(B,L) int → (B,C,L)."""
    B, C, L = x.shape
    W = weight.shape[1]
    xf = x.float()
    if seq_idx is None:
        y = F.conv1d(xf, weight.float().unsqueeze(1), None if bias is None else bias.float(), padding=W - 1,
                     groups=C)[..., :L]
    else:
        y = torch.zeros_like(xf)
        for j in range(W):
            shift = W - 1 - j
            xs = F.pad(xf, (shift, 0))[..., :L]
            ss = F.pad(seq_idx, (shift, 0), value=-1)[..., :L]
            same = (ss == seq_idx).unsqueeze(1)
            y = y + weight[:, j].float().view(1, C, 1) * xs * same
        if bias is not None:
            y = y + bias.float().view(1, C, 1)
    if activation in ("silu", "swish"):
        y = F.silu(y)
    return y.to(x.dtype)


def _rows(t: torch.Tensor) -> torch.Tensor:
    if t.stride(2) == 1 and t.stride(1) % 8 == 0 and (t.size(0) == 1 or t.stride(0) == t.size(1) * t.stride(1)) \
            and t.data_ptr() % 16 == 0:
        return t
    return t.contiguous()


class _ConvFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, seq_idx, silu):
        ext = backend.require_extension()
        x = _rows(x)
        wf = weight.float().contiguous()
        bf = None if bias is None else bias.float().contiguous()
        y = ext.causal_conv1d_fwd(x, wf, bf, seq_idx, silu)
        backend.count_launch()
        ctx.save_for_backward(x, wf, bf if bf is not None else torch.empty(0),
                              seq_idx if seq_idx is not None else torch.empty(0))
        ctx.silu, ctx.has_bias, ctx.has_seq = silu, bias is not None, seq_idx is not None
        ctx.wdtype, ctx.bdtype = weight.dtype, (None if bias is None else bias.dtype)
        return y

    @staticmethod
    def backward(ctx, dy):
        ext = backend.require_extension()
        x, wf, bf, seq_idx = ctx.saved_tensors
        dx, dw, db = ext.causal_conv1d_bwd(_rows(dy), x, wf, bf if ctx.has_bias else None,
                                           seq_idx if ctx.has_seq else None, ctx.silu)
        backend.count_launch()
        return dx, dw.to(ctx.wdtype), (db.to(ctx.bdtype) if ctx.has_bias else None), None, None


def causal_conv1d(x, weight, bias=None, seq_idx=None, activation: Optional[str] = None, channel_last: bool = False):
    """x:(B,C,L), or (B,L,C) when ``channel_last`` (the kernel's native layout); returns the same layout."""
    xl = x if channel_last else x.transpose(1, 2)
    if (backend.has("causal_conv1d_fwd") and xl.dtype in (torch.bfloat16, torch.float32) and 2 <= weight.shape[1] <= 4
            and xl.shape[-1] % 8 == 0 and backend.use_cuda_kernel("conv1d", xl, weight)):
        y = _ConvFn.apply(xl, weight, bias, None if seq_idx is None else seq_idx.to(torch.int32).contiguous(),
                          activation in ("silu", "swish"))
        return y if channel_last else y.transpose(1, 2)
    y = causal_conv1d_ref(xl.transpose(1, 2), weight, bias, seq_idx, activation)
    return y.transpose(1, 2) if channel_last else y
