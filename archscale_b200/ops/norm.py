"""RMSNorm / LayerNorm / gated RMSNorm.

Behavioural reference: `lit_gpt/rmsnorm.py:133-249` (oracles ``rms_norm_ref`` /
``layer_norm_ref``), `:1182-1215` (``FusedRMSNorm``), `lit_gpt/ops/layernorm_gated.py:18-39`
(gated oracle).  Statistics are always taken in fp32; the output has the input dtype.

CUDA path: ``csrc/norm.cu`` — one warp-group per row block, fp32 statistics, the saved
``rstd`` feeds a two-stage backward (per-CTA partial dw in fp32, then a column reduce).
"""
from __future__ import annotations

from typing import Optional

import torch

from . import backend


# ------------------------------------------------------------------ oracles
def rms_norm_ref(x: torch.Tensor, weight: Optional[torch.Tensor], eps: float = 1e-5,
                 residual: Optional[torch.Tensor] = None, prenorm: bool = False):
    dtype = x.dtype
    xf = x.float()
    if residual is not None:
        xf = xf + residual.float()
    rstd = torch.rsqrt(xf.pow(2).mean(dim=-1, keepdim=True) + eps)
    out = xf * rstd
    if weight is not None:
        out = out * weight.float()
    out = out.to(dtype)
    return (out, xf.to(residual.dtype if residual is not None else dtype)) if prenorm else out


def layer_norm_ref(x: torch.Tensor, weight: Optional[torch.Tensor], bias: Optional[torch.Tensor],
                   eps: float = 1e-5) -> torch.Tensor:
    dtype = x.dtype
    xf = x.float()
    mean = xf.mean(dim=-1, keepdim=True)
    var = xf.var(dim=-1, keepdim=True, correction=0)
    out = (xf - mean) * torch.rsqrt(var + eps)
    if weight is not None:
        out = out * weight.float()
    if bias is not None:
        out = out + bias.float()
    return out.to(dtype)


def gated_rms_norm_ref(x: torch.Tensor, weight: torch.Tensor, z: Optional[torch.Tensor], eps: float = 1e-5,
                       group_size: Optional[int] = None, norm_before_gate: bool = True) -> torch.Tensor:
    """``rmsnorm(x) * w * silu(z)`` (norm_before_gate) or ``rmsnorm(x * silu(z)) * w``, per group."""
    dtype = x.dtype
    xf = x.float()
    zf = z.float() if z is not None else None
    if zf is not None and not norm_before_gate:
        xf = xf * torch.nn.functional.silu(zf)
    n = xf.shape[-1]
    g = n if group_size is None else group_size
    xg = xf.reshape(*xf.shape[:-1], n // g, g)
    rstd = torch.rsqrt(xg.pow(2).mean(dim=-1, keepdim=True) + eps)
    out = (xg * rstd).reshape(xf.shape) * weight.float()
    if zf is not None and norm_before_gate:
        out = out * torch.nn.functional.silu(zf)
    return out.to(dtype)


# ------------------------------------------------------------------ CUDA autograd
class _RMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, eps, out_dtype):
        ext = backend.require_extension()
        shape = x.shape
        x2 = x.reshape(-1, shape[-1]).contiguous()
        out, rstd = ext.rmsnorm_fwd(x2, weight, eps, out_dtype)
        backend.count_launch()
        ctx.save_for_backward(x2, weight, rstd)
        ctx.shape = shape
        return out.view(shape)

    @staticmethod
    def backward(ctx, dout):
        ext = backend.require_extension()
        x2, weight, rstd = ctx.saved_tensors
        dout2 = dout.reshape(-1, ctx.shape[-1]).contiguous()
        dx, dw = ext.rmsnorm_bwd(dout2, x2, weight, rstd)
        backend.count_launch(2 if weight is not None else 1)
        return dx.view(ctx.shape), (dw.to(weight.dtype) if weight is not None else None), None, None


def rms_norm(x: torch.Tensor, weight: Optional[torch.Tensor], eps: float = 1e-5,
             out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """RMSNorm over the last dim; ``out_dtype`` (default: dtype of ``x``) lets the kernel read an fp32
    residual stream and write the bf16 mixer input in one pass."""
    ok_dtype = x.dtype in (torch.bfloat16, torch.float32) and (weight is None or weight.dtype in (torch.bfloat16, torch.float32))
    if ok_dtype and x.shape[-1] % 8 == 0 and x.shape[-1] <= 16384 and backend.use_cuda_kernel("rmsnorm", x, weight):
        return _RMSNormFn.apply(x, weight, eps, out_dtype)
    out = rms_norm_ref(x, weight, eps)
    return out if out_dtype is None else out.to(out_dtype)


class _LayerNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, eps):
        ext = backend.require_extension()
        x2 = x.reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        wf = None if weight is None else weight.float().contiguous()
        bf = None if bias is None else bias.float().contiguous()
        y, mean, rstd = ext.layernorm_fwd(x2, wf, bf, eps)
        backend.count_launch()
        ctx.save_for_backward(x2, wf if wf is not None else torch.empty(0), mean, rstd)
        ctx.has_w, ctx.has_b = weight is not None, bias is not None
        ctx.wdtype = None if weight is None else weight.dtype
        ctx.bdtype = None if bias is None else bias.dtype
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        ext = backend.require_extension()
        x2, wf, mean, rstd = ctx.saved_tensors
        dy2 = dy.reshape(x2.shape)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx, dw, db = ext.layernorm_bwd(dy2, x2, wf if ctx.has_w else None, mean, rstd)
        backend.count_launch(2)
        return (dx.view(dy.shape), dw.to(ctx.wdtype) if ctx.has_w else None, db.to(ctx.bdtype) if ctx.has_b else None, None)


def layer_norm(x: torch.Tensor, weight: Optional[torch.Tensor], bias: Optional[torch.Tensor],
               eps: float = 1e-5) -> torch.Tensor:
    """LayerNorm over the last dimension (`lit_gpt/rmsnorm.py:935-1096` with ``is_rms_norm=False``)."""
    if (x.is_cuda and x.dtype in (torch.bfloat16, torch.float32) and x.shape[-1] % 8 == 0 and x.shape[-1] <= 2560
            and backend.has("layernorm_fwd") and backend.use_cuda_kernel("layernorm", x)):
        return _LayerNormFn.apply(x, weight, bias, eps)
    return layer_norm_ref(x, weight, bias, eps)


class _GatedRMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, z, eps, gsize, nbg):
        ext = backend.require_extension()
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        z2 = None if z is None else z.reshape(-1, z.shape[-1]).contiguous()
        wf = weight.float().contiguous()
        y, rstd = ext.gated_rmsnorm_fwd(x2, z2, wf, eps, gsize, nbg)
        backend.count_launch()
        ctx.save_for_backward(x2, z2 if z2 is not None else torch.empty(0), wf, rstd)
        ctx.meta = (gsize, nbg, z is not None, weight.dtype, x.shape)
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        ext = backend.require_extension()
        x2, z2, wf, rstd = ctx.saved_tensors
        gsize, nbg, has_z, wdtype, shape = ctx.meta
        dx, dz, dw = ext.gated_rmsnorm_bwd(dy.reshape(x2.shape).contiguous(), x2, z2 if has_z else None, wf, rstd, gsize, nbg)
        backend.count_launch()
        return dx.view(shape), dw.to(wdtype), (dz.view(shape) if has_z else None), None, None, None


def gated_rms_norm(x, weight, z=None, eps: float = 1e-5, group_size: Optional[int] = None,
                   norm_before_gate: bool = True) -> torch.Tensor:
    """Gated RMSNorm with groups (`lit_gpt/ops/layernorm_gated.py:42-105,151-270`)."""
    n = x.shape[-1]
    g = n if group_size is None else group_size
    if (x.is_cuda and x.dtype in (torch.bfloat16, torch.float32) and (z is None or z.dtype == x.dtype) and g % 8 == 0 and n % g == 0
            and g <= 12288 and backend.has("gated_rmsnorm_fwd") and backend.use_cuda_kernel("gated_rmsnorm", x)):
        return _GatedRMSNormFn.apply(x, weight, z, eps, g, norm_before_gate)
    return gated_rms_norm_ref(x, weight, z, eps, group_size, norm_before_gate)


# ------------------------------------------------------------------ fused residual add + RMSNorm
def add_rms_norm_ref(res: torch.Tensor, h: Optional[torch.Tensor], weight: torch.Tensor, eps: float = 1e-5,
                     h_scale: float = 1.0, out_dtype: torch.dtype = torch.bfloat16,
                     stream_dtype: torch.dtype = torch.float32):
    """x = res + h_scale·h computed in fp32 and kept in ``stream_dtype``; returns (x, rmsnorm(x)·w in ``out_dtype``)."""
    x = res.float()
    if h is not None:
        x = x + h_scale * h.float()
    x = x.to(stream_dtype)
    return x, rms_norm_ref(x, weight, eps).to(out_dtype)


class _AddRMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, res, h, weight, eps, h_scale, bf16_stream):
        ext = backend.require_extension()
        shape = res.shape
        res2 = res.reshape(-1, shape[-1])
        h2 = h.reshape(-1, shape[-1]) if h is not None else None
        x, n, rstd = ext.add_rmsnorm_fwd(res2, h2, h_scale, weight, eps, bf16_stream)
        backend.count_launch()
        ctx.save_for_backward(x, weight, rstd)
        ctx.shape, ctx.h_scale, ctx.has_h, ctx.res_dtype, ctx.bf16_stream = shape, h_scale, h is not None, res.dtype, bf16_stream
        return x.view(shape), n.view(shape)

    @staticmethod
    def backward(ctx, g_x, g_n):
        ext = backend.require_extension()
        x, weight, rstd = ctx.saved_tensors
        C = ctx.shape[-1]
        if g_n is None:
            g_n = torch.zeros(x.shape, dtype=torch.bfloat16, device=x.device)
        g_n2 = g_n.reshape(-1, C)
        if not g_n2.is_contiguous():
            g_n2 = g_n2.contiguous()
        g_dtype = torch.bfloat16 if ctx.bf16_stream else torch.float32
        g_x2 = None
        if g_x is not None:
            g_x2 = g_x.reshape(-1, C)
            if g_x2.dtype != g_dtype or not g_x2.is_contiguous():
                g_x2 = g_x2.to(g_dtype).contiguous()
        d_res, d_h, dw = ext.add_rmsnorm_bwd(g_x2, g_n2, x, weight, rstd, ctx.has_h, ctx.h_scale, ctx.bf16_stream)
        backend.count_launch(2)
        if ctx.res_dtype != d_res.dtype:
            d_res = d_res.to(ctx.res_dtype)
        return d_res.view(ctx.shape), (d_h.view(ctx.shape) if ctx.has_h else None), dw.to(weight.dtype), None, None, None


def fused_cols_ok(cols: int) -> bool:
    """Row widths the fused residual-add + RMSNorm kernels take (register-resident weight-gradient accumulators)."""
    return cols % 8 == 0 and 512 <= cols <= 4096



def add_rms_norm(res: torch.Tensor, h: Optional[torch.Tensor], weight: torch.Tensor, eps: float = 1e-5,
                 h_scale: float = 1.0, out_dtype: torch.dtype = torch.bfloat16, stream_dtype: torch.dtype = torch.float32):
    """Pre-norm block entry: ``x = res + h_scale·h`` (the new residual stream, in ``stream_dtype``: fp32, or bf16 as the
    reference's bf16 mixed precision keeps it) and ``rmsnorm(x)·w``.

    One kernel forward; backward fuses the residual-gradient add, the RMSNorm backward and the bf16
    cast of the branch gradient."""
    bf16_stream = stream_dtype == torch.bfloat16 and res.dtype == torch.bfloat16
    if (fused_cols_ok(res.shape[-1]) and out_dtype == torch.bfloat16 and res.dtype in (torch.float32, torch.bfloat16)
            and (h is None or h.dtype == torch.bfloat16) and backend.has("add_rmsnorm_fwd")
            and backend.use_cuda_kernel("add_rmsnorm", res, h, weight)):
        return _AddRMSNormFn.apply(res.contiguous(), None if h is None else h.contiguous(), weight, eps, h_scale, bf16_stream)
    return add_rms_norm_ref(res, h, weight, eps, h_scale, out_dtype, stream_dtype)
