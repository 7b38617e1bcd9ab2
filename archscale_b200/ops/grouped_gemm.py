"""Mixture-of-experts FFN on the tcgen05 grouped GEMM (python side and autograd).

See :mod:`archscale_b200.ops.moe` for the semantics.  Data flow (all on the device, no host sync —
the reference copies token counts to the host every layer, `lit_gpt/moe.py:622-623`):

    indices ─► routing_layout ─► offsets (256-aligned expert segments), slot↔pair maps
    x ─► gather_rows ─► xs ─► grouped GEMM (W_in) ─► SwiGLU ─► grouped GEMM (W_out) ─► combine_rows(scores)

Backward runs the same pieces transposed: gate-weight gradients are row dot products, the
expert-weight gradients are grouped TN GEMMs whose K-loop walks each expert's row segment and
accumulates straight into the fp32 flat gradient buffer when the engine provides one.
"""
from __future__ import annotations

import torch

from . import backend
from .gemm import fused_swiglu_enabled


def supported(x, w_in, w_out, b_in, b_out) -> bool:
    if not x.is_cuda or b_in is not None or b_out is not None:
        return False
    if not backend.has("grouped_gemm_bf16"):
        return False
    C, I2, I = x.shape[1], w_in.shape[1], w_out.shape[2]
    return (x.dtype == torch.bfloat16 and w_in.dtype == torch.bfloat16 and w_out.dtype == torch.bfloat16
            and C % 64 == 0 and I2 % 64 == 0 and I % 64 == 0 and w_in.shape[0] <= 256)


class _MoEFFNFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w_in, w_out, scores, indices, shared=None, alpha=1.0):
        ext = backend.require_extension()
        N, C = x.shape
        E, I2, _ = w_in.shape
        I = w_out.shape[2]
        K = indices.shape[1]
        x = x.contiguous()
        sc = scores.float().contiguous()
        counts, offsets, slot_pair, pair_slot = ext.routing_layout(indices.reshape(-1).contiguous(), E)
        xs = ext.gather_rows(x, slot_pair, None, K, offsets)
        if xs.shape[0] % 256 == 0 and fused_swiglu_enabled():
            h, a = ext.grouped_gemm_swiglu(xs, w_in.reshape(E * I2, C), offsets, I, True)      # SwiGLU in the epilogue
        else:
            h = ext.grouped_gemm_bf16(0, xs, w_in.reshape(E * I2, C), offsets, 0, I2, C, None)
            a = ext.swiglu_packed_fwd(h)
        y = ext.grouped_gemm_bf16(0, a, w_out.reshape(E * C, I), offsets, 0, C, I, None)
        # out = alpha · (Σ_k score_k · y_k + shared): the shared expert's output and the mixing factor ride on the combine pass
        out = ext.combine_rows(y, pair_slot, sc, N, K, None if shared is None else shared.contiguous(), float(alpha))
        backend.count_launch(9)
        # `a` is kept as well (a quarter of the size of xs or y): recomputing it in backward is one more pass over h
        ctx.save_for_backward(xs, h, a, y, w_in, w_out, sc, offsets, slot_pair, pair_slot)
        ctx.dims = (N, C, E, I2, I, K)
        ctx.w_refs = (w_in, w_out)
        ctx.score_dtype = scores.dtype
        ctx.alpha = float(alpha)
        ctx.has_shared = shared is not None
        return out

    @staticmethod
    def backward(ctx, dout):
        ext = backend.require_extension()
        xs, h, a, y, w_in, w_out, sc, offsets, slot_pair, pair_slot = ctx.saved_tensors
        N, C, E, I2, I, K = ctx.dims
        dout = dout.contiguous()
        alpha = ctx.alpha
        dots = ext.pair_dots(y, dout, pair_slot, K).view(N, K)
        if alpha != 1.0:
            dots, sc = dots * alpha, sc * alpha                                        # [N, K] tensors: the factor costs no pass over rows
        dscores = dots.to(ctx.score_dtype)
        dy = ext.gather_rows(dout, slot_pair, sc.reshape(-1), K, offsets)             # dy[slot] = alpha · score · dout[token]
        da = ext.grouped_gemm_bf16(1, dy, w_out.reshape(E * C, I), offsets, 0, I, C, None)
        mg_out = getattr(ctx.w_refs[1], "main_grad", None)
        dw_out = ext.grouped_gemm_bf16(2, dy, a, offsets, C, I, 0, mg_out)
        dh = ext.swiglu_packed_bwd(h, da)
        dxs = ext.grouped_gemm_bf16(1, dh, w_in.reshape(E * I2, C), offsets, 0, C, I2, None)
        mg_in = getattr(ctx.w_refs[0], "main_grad", None)
        dw_in = ext.grouped_gemm_bf16(2, dh, xs, offsets, I2, C, 0, mg_in)
        dx = ext.combine_rows(dxs, pair_slot, None, N, K)
        backend.count_launch(8)
        dshared = None
        if ctx.has_shared:
            dshared = dout if alpha == 1.0 else dout * alpha
        return (dx, (None if mg_in is not None else dw_in), (None if mg_out is not None else dw_out), dscores, None,
                dshared, None)


def moe_ffn_cuda(x, w_in, w_out, scores, indices, shared=None, alpha=1.0):
    """alpha · (routed FFN + shared); ``shared`` (N, C) is the shared expert's output, if any."""
    return _MoEFFNFn.apply(x, w_in, w_out, scores, indices.to(torch.int32), shared, alpha)
