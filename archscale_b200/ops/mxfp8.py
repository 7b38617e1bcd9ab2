"""Block-scaled MXFP8 linear layers (OCP microscaling: e4m3 elements, one power-of-two E8M0 scale per 32
elements along the contraction dimension).

Replaces the ``te.Linear`` + ``MXFP8BlockScaling`` recipe of the reference (`precision.py:84-106,192-251`):
the master weight stays bf16/fp32; every GEMM of the layer quantises its operands on the fly:

* forward  ``y  = Q_row(x)  · Q_row(W)ᵀ``            (contraction over in_features)
* dgrad    ``dx = Q_row(dy) · Q_col(W)ᵀ``            (contraction over out_features; ``Q_col(W)`` is Wᵀ quantised)
* wgrad    ``dW = Q_col(dy) · Q_col(x)ᵀ``            (contraction over tokens), accumulated into fp32 ``main_grad``

``Q_row`` scales blocks along the stored rows, ``Q_col`` writes the transposed operand with blocks along the original
rows, so all three products are K-major "NT" GEMMs for ``tcgen05.mma.kind::mxf8f6f4.block_scale``
(``csrc/gemm_mxfp8.cu``).  Scale = smallest power of two ≥ amax/448, so quantisation never saturates.

The functions ending in ``_ref`` are plain PyTorch restatements used as the CPU path and as test oracles.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import backend

E4M3_MAX = 448.0


# ------------------------------------------------------------------------------------------------ references
def quantize_ref(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Row-wise MXFP8 of x:(R,K) → (q float8_e4m3fn (R,K), biased E8M0 exponents uint8 (R,K/32))."""
    R, K = x.shape
    xb = x.float().view(R, K // 32, 32)
    amax = xb.abs().amax(-1)
    v = amax / E4M3_MAX
    m, e = torch.frexp(v)                               # v = m·2^e, m in [0.5, 1)
    exp = torch.where(m == 0.5, e - 1, e)               # ceil(log2 v)
    biased = (exp + 127).clamp(1, 253).to(torch.int32)
    biased = torch.where(amax == 0, torch.ones_like(biased), biased)
    scale = torch.exp2((biased - 127).float())
    q = (xb / scale.unsqueeze(-1)).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn).view(R, K)
    return q, biased.to(torch.uint8)


def dequantize_ref(q: torch.Tensor, biased: torch.Tensor) -> torch.Tensor:
    R, K = q.shape
    return (q.float().view(R, K // 32, 32) * torch.exp2(biased.float() - 127).unsqueeze(-1)).view(R, K)


def chunk_scales_ref(biased: torch.Tensor) -> torch.Tensor:
    """(rows, K/32) exponents → the 512-byte-chunk order the kernels use (see ``csrc/gemm_mxfp8.cu``)."""
    rows, kb = biased.shape
    rp = (rows + 127) // 128 * 128
    full = torch.zeros(rp, kb, dtype=torch.uint8, device=biased.device)
    full[:rows] = biased
    # [chunk_r, m1(4), m0(32), chunk_k, k1(4)] → [chunk_r, chunk_k, m0, m1, k1]
    t = full.view(rp // 128, 4, 32, kb // 4, 4).permute(0, 3, 2, 1, 4).contiguous()
    return t.view(-1)


def unchunk_scales_ref(sf: torch.Tensor, rows: int, K: int) -> torch.Tensor:
    kb = K // 32
    rp = (rows + 127) // 128 * 128
    t = sf.view(rp // 128, kb // 4, 32, 4, 4).permute(0, 3, 2, 1, 4).contiguous().view(rp, kb)
    return t[:rows]


def linear_mxfp8_ref(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Forward of the MXFP8 linear in plain PyTorch (quantise → dequantise → fp32 matmul)."""
    x2 = x.reshape(-1, x.shape[-1])
    xq = dequantize_ref(*quantize_ref(x2))
    wq = dequantize_ref(*quantize_ref(weight))
    y = (xq @ wq.t()).to(x.dtype)
    if bias is not None:
        y = y + bias.to(y.dtype)
    return y.view(*x.shape[:-1], weight.shape[0])


# ------------------------------------------------------------------------------------------------ kernels
def quantize(x: torch.Tensor, colwise: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """x:(R,C) bf16 → (q uint8 e4m3 bits, chunked scales).  ``colwise`` returns the transposed operand (C,R)."""
    ext = backend.require_extension()
    backend.count_launch()
    return ext.mxfp8_quantize(x, colwise)


def quantize_both(x: torch.Tensor):
    """x:(R,C) bf16 → ((q, scales) row-wise, (qT, scales) of the transposed operand) from one read of x."""
    ext = backend.require_extension()
    backend.count_launch()
    q, sf, qt, sft = ext.mxfp8_quantize_both(x)
    return (q, sf), (qt, sft)


def gemm(a_q, a_sf, b_q, b_sf, out_f32: bool = False, acc: Optional[torch.Tensor] = None, alpha: float = 1.0):
    """``a_q:(M,K) · b_q:(N,K)ᵀ`` with block scales → (M,N) bf16 / fp32, or ``acc += …`` (fp32)."""
    ext = backend.require_extension()
    backend.count_launch()
    return ext.gemm_mxfp8(a_q, a_sf, b_q, b_sf, out_f32, acc, alpha)


def supported(x2: torch.Tensor, weight: torch.Tensor) -> bool:
    """Shapes the block-scaled kernels take: every contraction dimension a multiple of 128."""
    T, K = x2.shape
    N = weight.shape[0]
    return (x2.is_cuda and x2.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and K % 128 == 0 and N % 128 == 0
            and T % 128 == 0 and backend.has("gemm_mxfp8"))


# Quantised weights are reused until the weights change: a forward under activation checkpointing runs twice and every
# micro-step of a gradient-accumulation window sees the same values.  The optimizer step (and a checkpoint load) call
# ``invalidate_weight_cache()``; an entry is also dropped when the tensor's storage or in-place version moved.
_W_EPOCH = 0
_W_CACHE: dict = {}


def invalidate_weight_cache() -> None:
    global _W_EPOCH
    _W_EPOCH += 1
    _W_CACHE.clear()


def quantize_weight(weight: torch.Tensor, colwise: bool) -> Tuple[torch.Tensor, torch.Tensor]:
    key = (id(weight), colwise)
    tag = (_W_EPOCH, weight.data_ptr(), weight._version, tuple(weight.shape))
    hit = _W_CACHE.get(key)
    if hit is not None and hit[0] == tag:
        return hit[1]
    out = quantize(weight, colwise)
    _W_CACHE[key] = (tag, out)
    return out


class _LinearMXFP8Fn(torch.autograd.Function):
    """A tensor needed in both orientations is read once: x is quantised row-wise (forward product) and transposed (weight
    gradient; saved in place of x itself) by one kernel, and so is dy in the backward pass (dgrad and wgrad)."""

    @staticmethod
    def forward(ctx, x, weight, bias):
        x2 = x.reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        if ctx.needs_input_grad[1]:
            (xq, xs), xt = quantize_both(x2)
            ctx.save_for_backward(weight, *xt)
        else:
            xq, xs = quantize(x2)
            ctx.save_for_backward(weight)
        wq, ws = quantize_weight(weight, False)
        y = gemm(xq, xs, wq, ws)
        if bias is not None:
            y = y + bias.to(y.dtype)
        ctx.has_bias = bias is not None
        ctx.weight_ref = weight
        ctx.x_shape = x.shape
        return y.view(*x.shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, dy):
        weight, *xt = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = dw = db = None
        need_dx, need_dw = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        if need_dx and need_dw:
            g, gt = quantize_both(dy2)                      # (T, N) blocks along N; dyᵀ: (N, T) blocks along T
        elif need_dx:
            g, gt = quantize(dy2), None
        else:
            g, gt = None, quantize(dy2, colwise=True)
        if need_dx:
            wtq, wts = quantize_weight(weight, True)        # Wᵀ: (K, N) blocks along N
            dx = gemm(g[0], g[1], wtq, wts).view(ctx.x_shape)
        if need_dw:
            xtq, xts = xt                                   # xᵀ : (K, T) blocks along T
            main_grad = getattr(ctx.weight_ref, "main_grad", None)
            if main_grad is not None:
                gemm(gt[0], gt[1], xtq, xts, acc=main_grad)
            else:
                dw = gemm(gt[0], gt[1], xtq, xts).to(weight.dtype)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy2.float().sum(0).to(dy.dtype)
        return dx, dw, db


def linear_mxfp8(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """MXFP8 ``x @ weightᵀ + bias``; shapes the kernels do not take (or CPU tensors) run in bf16 / fp32."""
    x2 = x.reshape(-1, x.shape[-1])
    if supported(x2, weight) and backend.use_cuda_kernel("mxfp8", x2, weight):
        return _LinearMXFP8Fn.apply(x, weight, bias)
    from .gemm import linear
    return linear(x, weight, bias)
