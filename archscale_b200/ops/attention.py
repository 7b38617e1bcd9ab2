"""Causal / sliding-window / packed-varlen attention with GQA, returning the log-sum-exp.

Semantics follow the flash-attention call the reference makes
(`lit_gpt/attention.py:63-68,121,347-424`): layout ``(B, T, H, D)``, causal, optional
left window ``(w-1, 0)`` (query ``i`` sees keys ``i-w+1 .. i``), optional ``cu_seqlens``
(documents packed in one row never attend across a boundary), K/V with ``G`` heads shared
by ``H/G`` query heads, optional learnable per-head sink logit (softmax denominator gets
an extra ``exp(sink)`` term, `lit_gpt/oss_attn.py:186-197`).

CUDA path: ``csrc/attention.cu`` — tcgen05 QKᵀ and PV with S/P/O accumulators in TMEM,
K/V tiles streamed by TMA, online softmax in registers; backward recomputes P from the
saved LSE and accumulates dQ deterministically.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

from . import backend


def _build_mask(Tq: int, Tk: int, device, window: Tuple[int, int], cu_seqlens: Optional[torch.Tensor]):
    """Boolean (Tq, Tk) mask, True = may attend.  Queries are aligned to the end of the keys."""
    qi = torch.arange(Tq, device=device).unsqueeze(1) + (Tk - Tq)
    kj = torch.arange(Tk, device=device).unsqueeze(0)
    allowed = kj <= qi
    if window[0] >= 0:
        allowed &= kj >= qi - window[0]
    if cu_seqlens is not None:
        pos = torch.arange(Tk, device=device)
        seg = torch.bucketize(pos, cu_seqlens[1:].to(device), right=True)
        allowed &= seg[Tk - Tq:].unsqueeze(1) == seg.unsqueeze(0)
    return allowed


def attention_ref(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: Optional[float] = None,
                  window: Tuple[int, int] = (-1, -1), cu_seqlens: Optional[torch.Tensor] = None,
                  sink: Optional[torch.Tensor] = None, return_lse: bool = False):
    """fp32 dense-softmax oracle.  q:(B,Tq,H,D) k,v:(B,Tk,G,D)."""
    B, Tq, H, D = q.shape
    Tk, G = k.shape[1], k.shape[2]
    scale = 1.0 / math.sqrt(D) if scale is None else scale
    qf = q.float().permute(0, 2, 1, 3)                                      # B H Tq D
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(H // G, dim=1)     # B H Tk D
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(H // G, dim=1)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    mask = _build_mask(Tq, Tk, q.device, window, cu_seqlens)
    s = s.masked_fill(~mask, float("-inf"))
    if sink is not None:
        s = torch.cat((s, sink.float().view(1, H, 1, 1).expand(B, H, Tq, 1)), dim=-1)
    lse = torch.logsumexp(s, dim=-1)                                        # B H Tq
    p = torch.exp(s - lse.unsqueeze(-1))
    if sink is not None:
        p = p[..., :-1]
    o = torch.matmul(p, vf).permute(0, 2, 1, 3).to(q.dtype)
    return (o, lse) if return_lse else o


def pointwise_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, kind: str, scale: Optional[float] = None,
                        window: Tuple[int, int] = (-1, -1), cu_seqlens: Optional[torch.Tensor] = None,
                        sigmoid_bias: float = 0.0, q_chunk: int = 1024) -> torch.Tensor:
    """The two attention variants of the reference that are not softmax-weighted sums, as query-chunked PyTorch math
    (memory O(q_chunk · Tk) per head; both are small-scale options of the reference, not hot paths):

    * ``kind="sigmoid"`` — ``Σ_j sigmoid(scale·q_i·k_j + bias)·v_j`` over the causal (windowed, per-document) keys: what
      ``flash_sigmoid.flash_attn_func(..., sigmoid_bias=0)`` computes at `lit_gpt/attention.py:353-356`;
    * ``kind="sqrt_softmax"`` — ``sqrt(softmax(scale·q kᵀ + causal mask) + 1e-5) @ silu(v)``, the non-``fa2`` path at
      `lit_gpt/attention.py:426-441`.
    q:(B,Tq,H,D) k,v:(B,Tk,G,D) → (B,Tq,H,D)."""
    B, Tq, H, D = q.shape
    Tk, G = k.shape[1], k.shape[2]
    scale = 1.0 / math.sqrt(D) if scale is None else scale
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(H // G, dim=1)     # B H Tk D
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(H // G, dim=1)
    if kind == "sqrt_softmax":
        vf = torch.nn.functional.silu(vf)
    mask = _build_mask(Tq, Tk, q.device, window, cu_seqlens)                 # Tq × Tk, True = visible
    outs = []
    for s0 in range(0, Tq, q_chunk):
        qf = q[:, s0:s0 + q_chunk].float().permute(0, 2, 1, 3)              # B H c D
        logits = torch.matmul(qf, kf.transpose(-1, -2)) * scale
        m = mask[s0:s0 + q_chunk]
        if kind == "sigmoid":
            w = torch.sigmoid(logits + sigmoid_bias).masked_fill(~m, 0.0)
        elif kind == "sqrt_softmax":
            # as in the reference, the 1e-5 sits inside the root for every key, masked ones included (weight 0.0032 each)
            w = torch.sqrt(torch.softmax(logits.masked_fill(~m, float("-inf")), dim=-1) + 1e-5)
        else:
            raise ValueError(kind)
        outs.append(torch.matmul(w, vf))
    return torch.cat(outs, dim=2).permute(0, 2, 1, 3).to(q.dtype)


def row_start_from_cu_seqlens(cu_seqlens: torch.Tensor, total: int) -> torch.Tensor:
    """int32 (total,) first token of the document each position belongs to (device op, no host sync)."""
    pos = torch.arange(total, device=cu_seqlens.device)
    seg = torch.bucketize(pos, cu_seqlens[1:].to(pos.dtype), right=True)
    return cu_seqlens.to(torch.int32)[seg.clamp_max(cu_seqlens.numel() - 2)].contiguous()


def _sdpa_fallback(q, k, v, scale, window, cu_seqlens):
    """Library path used only when the extension is explicitly disabled on a GPU."""
    B, Tq, H, D = q.shape
    G = k.shape[2]
    if window[0] < 0 and cu_seqlens is None and Tq == k.shape[1]:
        o = torch.nn.functional.scaled_dot_product_attention(
            q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True, scale=scale,
            enable_gqa=(H != G))
        return o.transpose(1, 2)
    mask = _build_mask(Tq, k.shape[1], q.device, window, cu_seqlens)
    o = torch.nn.functional.scaled_dot_product_attention(
        q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), attn_mask=mask, scale=scale,
        enable_gqa=(H != G))
    return o.transpose(1, 2)


def doc_end_from_cu_seqlens(cu_seqlens: torch.Tensor, total: int) -> torch.Tensor:
    """int32 (total,) exclusive end of the document each position belongs to."""
    pos = torch.arange(total, device=cu_seqlens.device)
    seg = torch.bucketize(pos, cu_seqlens[1:].to(pos.dtype), right=True)
    return cu_seqlens.to(torch.int32)[(seg + 1).clamp_max(cu_seqlens.numel() - 1)].contiguous()


class _AttnFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, scale, window_left, cu_seqlens):
        ext = backend.require_extension()
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        row_start = doc_end = None
        if cu_seqlens is not None:
            T = q.shape[1]
            row_start, doc_end = row_start_from_cu_seqlens(cu_seqlens, T), doc_end_from_cu_seqlens(cu_seqlens, T)
        out, lse = ext.attn_fwd(q, k, v, scale, window_left, row_start)
        backend.count_launch()
        none = torch.empty(0)
        ctx.save_for_backward(q, k, v, out, lse, row_start if row_start is not None else none,
                              doc_end if doc_end is not None else none)
        ctx.scale, ctx.window_left, ctx.varlen = scale, window_left, cu_seqlens is not None
        ctx.mark_non_differentiable(lse)
        return out, lse

    @staticmethod
    def backward(ctx, dout, _dlse):
        ext = backend.require_extension()
        q, k, v, out, lse, row_start, doc_end = ctx.saved_tensors
        dq, dk, dv = ext.attn_bwd(dout.contiguous(), q, k, v, out, lse, ctx.scale, ctx.window_left,
                                  row_start if ctx.varlen else None, doc_end if ctx.varlen else None)
        backend.count_launch(3)
        return dq, dk, dv, None, None, None


class _AttnSinkFn(torch.autograd.Function):
    """Attention with a learnable per-head sink logit on the same kernels.  The sink adds ``exp(sink)`` to every softmax
    denominator and nothing to the numerator, so with ``lse`` the plain log-sum-exp: ``lse' = logaddexp(lse, sink)`` and
    ``out' = out · exp(lse − lse')``.  The backward kernels recompute the probabilities from the saved log-sum-exp and δ
    from ``dO·O``, so given (out', lse') they return the sink-softmax gradients unchanged; the sink column itself gets
    ``d sink_h = −Σ_{b,t} p_sink · δ`` with ``p_sink = exp(sink − lse')``."""

    @staticmethod
    def forward(ctx, q, k, v, sink, scale, window_left, cu_seqlens):
        ext = backend.require_extension()
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        row_start = doc_end = None
        if cu_seqlens is not None:
            T = q.shape[1]
            row_start, doc_end = row_start_from_cu_seqlens(cu_seqlens, T), doc_end_from_cu_seqlens(cu_seqlens, T)
        out, lse = ext.attn_fwd(q, k, v, scale, window_left, row_start)                 # lse: (B,H,T)
        backend.count_launch()
        sk = sink.float().view(1, -1, 1)
        lse_s = torch.logaddexp(lse, sk)
        keep = torch.exp(lse - lse_s)                                                   # share of the real keys
        out_s = (out.float() * keep.permute(0, 2, 1).unsqueeze(-1)).to(out.dtype)
        none = torch.empty(0)
        ctx.save_for_backward(q, k, v, out_s, lse_s, sink, row_start if row_start is not None else none,
                              doc_end if doc_end is not None else none)
        ctx.scale, ctx.window_left, ctx.varlen = scale, window_left, cu_seqlens is not None
        ctx.mark_non_differentiable(lse_s)
        return out_s, lse_s

    @staticmethod
    def backward(ctx, dout, _dlse):
        ext = backend.require_extension()
        q, k, v, out_s, lse_s, sink, row_start, doc_end = ctx.saved_tensors
        dout = dout.contiguous()
        dq, dk, dv = ext.attn_bwd(dout, q, k, v, out_s, lse_s, ctx.scale, ctx.window_left,
                                  row_start if ctx.varlen else None, doc_end if ctx.varlen else None)
        backend.count_launch(3)
        delta = (dout.float() * out_s.float()).sum(-1).permute(0, 2, 1)                 # (B,H,T)
        p_sink = torch.exp(sink.float().view(1, -1, 1) - lse_s)
        dsink = -(p_sink * delta).sum((0, 2))
        return dq, dk, dv, dsink.to(sink.dtype).view(sink.shape), None, None, None


def cuda_supported(q, k, v, sink) -> bool:
    D = q.shape[-1]
    return (backend.has("attn_fwd") and backend.has("attn_bwd") and q.dtype == torch.bfloat16 and k.dtype == torch.bfloat16
            and v.dtype == torch.bfloat16 and D in (64, 128) and v.shape[-1] == D and q.shape[1] == k.shape[1]
            and q.shape[2] % k.shape[2] == 0)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: Optional[float] = None,
              window: Tuple[int, int] = (-1, -1), cu_seqlens: Optional[torch.Tensor] = None,
              sink: Optional[torch.Tensor] = None, return_lse: bool = False):
    scale = 1.0 / math.sqrt(q.shape[-1]) if scale is None else scale
    if q.is_cuda and cuda_supported(q, k, v, sink) and backend.use_cuda_kernel("attention", q, k, v):
        if cu_seqlens is not None:
            assert q.shape[0] == 1, "packed varlen attention expects batch 1"
            cu_seqlens = cu_seqlens.to(torch.int32).contiguous()
        if sink is not None:
            out, lse = _AttnSinkFn.apply(q, k, v, sink, float(scale), int(window[0]), cu_seqlens)
        else:
            out, lse = _AttnFn.apply(q, k, v, float(scale), int(window[0]), cu_seqlens)
        return (out, lse) if return_lse else out
    if q.is_cuda and sink is None and not return_lse:
        return _sdpa_fallback(q, k, v, scale, window, cu_seqlens)
    return attention_ref(q, k, v, scale, window, cu_seqlens, sink, return_lse)
