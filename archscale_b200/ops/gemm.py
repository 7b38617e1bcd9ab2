"""Dense GEMM entry points and the ``linear`` autograd op built on them.

Three operand layouts cover forward, dgrad and wgrad of ``y = x @ Wᵀ``
(``nn.Linear`` everywhere in the reference, e.g. `lit_gpt/attention.py:42-48`,
`lit_gpt/model.py:636-637`):

* ``matmul_nt(a[M,K], b[N,K])  = a @ bᵀ``  (forward; both operands K-major)
* ``matmul_nn(a[M,K], b[K,N])  = a @ b``   (dgrad; B is N-major)
* ``matmul_tn(a[K,M], b[K,N])  = aᵀ @ b``  (wgrad; both operands MN-major)

CUDA path: ``csrc/gemm2_bf16.cu`` by default — SM pairs (``cta_group::2``) share one 256×256
output tile: each CTA loads its half of both operands with TMA, the leader's elected thread
issues ``tcgen05.mma`` for the pair into double-buffered TMEM accumulators, epilogue warps of
both CTAs drain their 128 rows with ``tcgen05.ld``.  ``csrc/gemm_bf16.cu`` is the one-CTA
kernel of the same structure (128×256 tiles), kept for shapes the pair kernel does not take and
selectable with ``ARCHSCALE_B200_GEMM=1cta``.  All three layouts run the same kernels with
different TMA boxes and UMMA descriptor major-ness.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import backend


def _cuda_ok(a: torch.Tensor, b: torch.Tensor, M: int, N: int, K: int) -> bool:
    return (a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16 and K % 8 == 0 and N % 8 == 0 and M % 8 == 0
            and K >= 64 and M >= 1 and a.dim() == 2 and b.dim() == 2
            and a.stride(-1) == 1 and b.stride(-1) == 1
            and a.stride(0) % 8 == 0 and b.stride(0) % 8 == 0
            and a.data_ptr() % 16 == 0 and b.data_ptr() % 16 == 0)


def matmul_nt(a: torch.Tensor, b: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """a:(M,K) b:(N,K) → a @ bᵀ : (M,N)."""
    M, K = a.shape
    N = b.shape[0]
    if _cuda_ok(a, b, M, N, K) and backend.use_cuda_kernel("gemm", a, b):
        backend.count_launch()
        return backend.require_extension().gemm_bf16(a, b, 0, out_dtype or torch.bfloat16, None)
    out = a @ b.t()
    return out if out_dtype is None else out.to(out_dtype)


def matmul_nn(a: torch.Tensor, b: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """a:(M,K) b:(K,N) → a @ b : (M,N)."""
    M, K = a.shape
    N = b.shape[1]
    if _cuda_ok(a, b, M, N, K) and backend.use_cuda_kernel("gemm", a, b):
        backend.count_launch()
        return backend.require_extension().gemm_bf16(a, b, 1, out_dtype or torch.bfloat16, None)
    out = a @ b
    return out if out_dtype is None else out.to(out_dtype)


def matmul_tn(a: torch.Tensor, b: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """a:(K,M) b:(K,N) → aᵀ @ b : (M,N)."""
    K, M = a.shape
    N = b.shape[1]
    if _cuda_ok(a, b, M, N, K) and backend.use_cuda_kernel("gemm", a, b):
        backend.count_launch()
        return backend.require_extension().gemm_bf16(a, b, 2, out_dtype or torch.bfloat16, None)
    out = a.t() @ b
    return out if out_dtype is None else out.to(out_dtype)


def matmul_tn_acc_(c: torch.Tensor, a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """c (fp32, (M,N)) += aᵀ @ b with a:(K,M), b:(K,N)."""
    K, M = a.shape
    N = b.shape[1]
    if c.dtype == torch.float32 and c.is_contiguous() and _cuda_ok(a, b, M, N, K) and backend.use_cuda_kernel("gemm", a, b, c):
        backend.count_launch()
        backend.require_extension().gemm_bf16(a, b, 2, torch.float32, c)
        return c
    if a.is_cuda:
        c.add_((a.t() @ b).to(c.dtype))
    else:
        c.add_(a.float().t() @ b.float())
    return c


class _LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias):
        ctx.save_for_backward(x, weight)
        ctx.has_bias = bias is not None
        ctx.weight_ref = weight            # to find ``main_grad`` (fp32 flat-buffer view) in backward
        x2 = x.reshape(-1, x.shape[-1])
        g = getattr(weight, "_fsdp_group", None)
        if g is not None and getattr(g, "ag_pending", False):
            eng = weight._fsdp_engine
            if weight._fsdp_first and _cuda_ok(x2, weight, x2.shape[0], weight.shape[0], x2.shape[1]):
                # FSDP forward: this GEMM also gathers the unit's matrix parameters from all ranks
                g.ag_pending = False
                y = eng.symm.ag_gemm(x2, g, weight.shape[0])
            else:
                eng.finish_pending_gather(g)
                y = matmul_nt(x2, weight)
        else:
            y = matmul_nt(x2, weight)
        if bias is not None:
            y = y + bias.to(y.dtype)
        return y.view(*x.shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x, weight = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        x2 = x.reshape(-1, x.shape[-1])
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = matmul_nn(dy2, weight).view(x.shape)
        if ctx.needs_input_grad[1]:
            main_grad = getattr(ctx.weight_ref, "main_grad", None)
            if main_grad is not None:
                matmul_tn_acc_(main_grad, dy2, x2)      # wgrad accumulates straight into fp32
            else:
                dw = matmul_tn(dy2, x2)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy2.float().sum(0).to(dy.dtype)
        return dx, dw, db


class _LinearSwiGLUFn(torch.autograd.Function):
    """``silu(x·W_gateᵀ) ∘ (x·W_upᵀ)`` with the activation computed in the GEMM epilogue (``W = [gate rows | up rows]``).
    The pre-activation is still written (the backward needs it) but not read back in the forward pass."""

    @staticmethod
    def forward(ctx, x, weight):
        x2 = x.reshape(-1, x.shape[-1])
        h, act = backend.require_extension().gemm_swiglu(x2, weight, True)
        backend.count_launch()
        ctx.save_for_backward(x, weight, h)
        ctx.weight_ref = weight
        return act.view(*x.shape[:-1], weight.shape[0] // 2)

    @staticmethod
    def backward(ctx, dact):
        x, weight, h = ctx.saved_tensors
        da2 = dact.reshape(-1, dact.shape[-1])
        if not da2.is_contiguous():
            da2 = da2.contiguous()
        dh = backend.require_extension().swiglu_packed_bwd(h, da2)
        backend.count_launch()
        x2 = x.reshape(-1, x.shape[-1])
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = matmul_nn(dh, weight).view(x.shape)
        if ctx.needs_input_grad[1]:
            main_grad = getattr(ctx.weight_ref, "main_grad", None)
            if main_grad is not None:
                matmul_tn_acc_(main_grad, dh, x2)
            else:
                dw = matmul_tn(dh, x2)
        return dx, dw


def fused_swiglu_enabled() -> bool:
    """SwiGLU in the epilogue of the SM-pair GEMM (off with ``ARCHSCALE_B200_FUSED_SWIGLU=0`` or the one-CTA GEMM)."""
    import os
    return (os.environ.get("ARCHSCALE_B200_FUSED_SWIGLU", "1") != "0" and os.environ.get("ARCHSCALE_B200_GEMM", "") != "1cta"
            and backend.has("gemm_swiglu"))


def linear_swiglu(x: torch.Tensor, weight: torch.Tensor) -> Optional[torch.Tensor]:
    """SwiGLU of ``x @ weightᵀ`` (gate = first half of the output features) in one GEMM launch, or ``None`` when the
    fused kernel does not take this case (the caller then runs ``linear`` + ``swiglu_packed``)."""
    if not (x.is_cuda and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and weight.dim() == 2
            and weight.shape[0] % 16 == 0 and x.shape[-1] % 8 == 0 and x.shape[-1] >= 64
            and (x.numel() // x.shape[-1]) % 8 == 0 and weight.stride(-1) == 1 and weight.stride(0) % 8 == 0
            and weight.data_ptr() % 16 == 0 and fused_swiglu_enabled() and backend.use_cuda_kernel("gemm", x, weight)):
        return None
    g = getattr(weight, "_fsdp_group", None)
    if g is not None and getattr(g, "ag_pending", False):
        return None                                     # this GEMM carries the unit's fused all-gather: keep that path
    if not x.is_contiguous():
        x = x.contiguous()
    return _LinearSwiGLUFn.apply(x, weight)


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x @ weightᵀ + bias``; bf16 CUDA inputs run the tcgen05 kernel for fwd, dgrad and wgrad."""
    if (x.is_cuda and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16
            and x.shape[-1] % 8 == 0 and weight.shape[0] % 8 == 0 and x.shape[-1] >= 64
            and (x.numel() // x.shape[-1]) % 8 == 0
            and backend.use_cuda_kernel("gemm", x, weight)):
        if not x.is_contiguous():
            x = x.contiguous()
        return _LinearFn.apply(x, weight, bias)
    g = getattr(weight, "_fsdp_group", None)
    if g is not None and getattr(g, "ag_pending", False):
        weight._fsdp_engine.finish_pending_gather(g)
    if weight.dtype != x.dtype:
        weight = weight.to(x.dtype)
        bias = bias.to(x.dtype) if bias is not None else None
    return torch.nn.functional.linear(x, weight, bias)


# ------------------------------------------------------------------------------------------ fused sibling projections
def _adjacent(ts) -> bool:
    """True when the tensors are dense 2-D row blocks stored back to back (views of one flat parameter buffer)."""
    for a, b in zip(ts[:-1], ts[1:]):
        if not (a.is_contiguous() and b.is_contiguous() and a.dtype == b.dtype and a.shape[1] == b.shape[1]
                and a.data_ptr() + a.numel() * a.element_size() == b.data_ptr()):
            return False
    return True


def _cat_view(ts) -> torch.Tensor:
    rows = sum(t.shape[0] for t in ts)
    return ts[0].as_strided((rows, ts[0].shape[1]), (ts[0].shape[1], 1))


class _MultiLinearFn(torch.autograd.Function):
    """y = x @ [W₀; W₁; …]ᵀ for weights stored back to back: one forward GEMM, one dgrad GEMM (no partial-sum adds) and
    one wgrad GEMM that accumulates into the equally adjacent fp32 ``main_grad`` views."""

    @staticmethod
    def forward(ctx, x, *weights):
        w_cat = _cat_view([w.detach() for w in weights])
        x2 = x.reshape(-1, x.shape[-1])
        g = getattr(weights[0], "_fsdp_group", None)
        if g is not None and getattr(g, "ag_pending", False):
            eng = weights[0]._fsdp_engine
            if weights[0]._fsdp_first and _cuda_ok(x2, w_cat, x2.shape[0], w_cat.shape[0], x2.shape[1]):
                g.ag_pending = False
                y = eng.symm.ag_gemm(x2, g, w_cat.shape[0])
            else:
                eng.finish_pending_gather(g)
                y = matmul_nt(x2, w_cat)
        else:
            y = matmul_nt(x2, w_cat)
        ctx.save_for_backward(x2, w_cat)
        ctx.weights = weights
        return y.view(*x.shape[:-1], w_cat.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w_cat = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = matmul_nn(dy2, w_cat).view(*dy.shape[:-1], x2.shape[1]) if ctx.needs_input_grad[0] else None
        mgs = [getattr(w, "main_grad", None) for w in ctx.weights]
        if all(m is not None for m in mgs) and _adjacent(mgs):
            matmul_tn_acc_(_cat_view(mgs), dy2, x2)
            return (dx,) + (None,) * len(ctx.weights)
        dw = matmul_tn(dy2, x2)
        outs, r = [], 0
        for w, m in zip(ctx.weights, mgs):
            piece = dw[r:r + w.shape[0]]
            r += w.shape[0]
            if m is not None:
                m.add_(piece.float())
                outs.append(None)
            else:
                outs.append(piece)
        return (dx,) + tuple(outs)


def linear_multi(x: torch.Tensor, layers, keep_fused: bool = False):
    """Outputs of several bias-free ``Linear`` layers that share the input ``x``.  When their weights sit back to back in
    memory (consecutive views of the flat parameter buffer) the layers run as one GEMM and the outputs are column
    slices of its result; otherwise each layer is called on its own.  ``keep_fused``: return the one GEMM's result unsplit
    (a tensor instead of a list) when the layers did run as one GEMM."""
    ws = [l.weight for l in layers]
    fusable = (x.is_cuda and x.dtype == torch.bfloat16 and all(type(l).__name__ == "Linear" and l.bias is None and not l.mxfp8
                                                              and not getattr(l, "nvfp4", False) for l in layers)
               and all(w.dtype == torch.bfloat16 for w in ws) and _adjacent(ws)
               and (x.numel() // x.shape[-1]) % 8 == 0 and x.shape[-1] % 8 == 0 and x.shape[-1] >= 64
               and backend.use_cuda_kernel("gemm", x, ws[0]))
    if not fusable:
        return [l(x) for l in layers]
    y = _MultiLinearFn.apply(x if x.is_contiguous() else x.contiguous(), *ws)
    if keep_fused:
        return y
    return list(y.split([w.shape[0] for w in ws], dim=-1))
