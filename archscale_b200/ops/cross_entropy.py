"""Cross-entropy and the fused linear + cross-entropy (FLCE) loss.

Behavioural reference: `lit_gpt/fused_cross_entropy.py:29-150` (label smoothing, z-loss,
ignore_index) and `lit_gpt/fused_linear_cross_entropy.py:36-143` (never materialise the
``[N, V]`` logits: process row chunks, compute the logits gradient in place and fold it
straight into ``dX`` and an fp32 ``dW`` accumulator).

Differences from the reference, on purpose: the chunk count adapts to ``V/H`` instead of a
fixed 8, no fp32 copy of the weight is made, and there is no host synchronisation (the
non-ignored-token count stays on the device).

CUDA path: logits chunk by the tcgen05 GEMM (``csrc/gemm_bf16.cu``), then
``csrc/cross_entropy.cu`` does online-softmax LSE + loss + in-place dlogits in one pass
over the chunk, then two more GEMMs produce ``dX_c`` and accumulate ``dW`` in fp32.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F

from . import backend
from . import gemm as _gemm


def cross_entropy_ref(logits: torch.Tensor, target: torch.Tensor, ignore_index: int = -100,
                      label_smoothing: float = 0.0, lse_square_scale: float = 0.0,
                      reduction: str = "mean") -> torch.Tensor:
    lf = logits.float()
    loss = F.cross_entropy(lf, target, ignore_index=ignore_index, label_smoothing=label_smoothing,
                           reduction="none")
    if lse_square_scale > 0:
        z = torch.logsumexp(lf, dim=-1).pow(2) * lse_square_scale
        loss = loss + z.masked_fill(target == ignore_index, 0.0)
    if reduction == "none":
        return loss
    n = (target != ignore_index).sum().clamp_min(1)
    return loss.sum() / n if reduction == "mean" else loss.sum()


def _ce_chunk_fwd_bwd(logits: torch.Tensor, target: torch.Tensor, ignore_index: int, label_smoothing: float,
                      lse_square_scale: float):
    """Returns (per-row loss fp32, dlogits with the same dtype as logits, written in place when possible).

    dlogits is d(sum of row losses)/dlogits; the caller scales by 1/n_valid.
    """
    if (logits.dtype in (torch.bfloat16, torch.float32) and logits.is_contiguous()
            and backend.use_cuda_kernel("cross_entropy", logits, target)):
        ext = backend.require_extension()
        loss = ext.cross_entropy_fwd_bwd_(logits, target, ignore_index, label_smoothing, lse_square_scale)
        backend.count_launch()
        return loss, logits
    lf = logits.float()
    lse = torch.logsumexp(lf, dim=-1, keepdim=True)
    p = torch.exp(lf - lse)
    valid = (target != ignore_index)
    tgt = target.clamp_min(0).unsqueeze(1)
    V = lf.shape[-1]
    nll = (lse - lf.gather(1, tgt)).squeeze(1)
    grad = p.clone()
    if label_smoothing > 0:
        smooth = (lse.squeeze(1) - lf.mean(dim=-1))
        loss = (1 - label_smoothing) * nll + label_smoothing * smooth
        grad.sub_(label_smoothing / V)
        grad.scatter_add_(1, tgt, torch.full_like(tgt, -(1 - label_smoothing), dtype=grad.dtype))
    else:
        loss = nll
        grad.scatter_add_(1, tgt, torch.full_like(tgt, -1.0, dtype=grad.dtype))
    if lse_square_scale > 0:
        loss = loss + lse_square_scale * lse.squeeze(1).pow(2)
        grad.add_(p * (2 * lse_square_scale * lse))
    loss = loss.masked_fill(~valid, 0.0)
    grad.mul_(valid.unsqueeze(1))
    return loss, grad.to(logits.dtype)


class _FLCEFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, target, ignore_index, label_smoothing, lse_square_scale, chunk_rows):
        N, H = x.shape
        V = weight.shape[0]
        need_dx = x.requires_grad
        need_dw = weight.requires_grad
        dx = torch.empty_like(x) if need_dx else None
        dw = torch.zeros(V, H, device=x.device, dtype=torch.float32) if need_dw else None
        total = torch.zeros((), device=x.device, dtype=torch.float32)
        n_valid = (target != ignore_index).sum().clamp_min(1).to(torch.float32)
        for s in range(0, N, chunk_rows):
            e = min(s + chunk_rows, N)
            xc = x[s:e]
            logits = _gemm.matmul_nt(xc, weight)                     # (rows, V), x dtype
            loss_rows, dlogits = _ce_chunk_fwd_bwd(logits, target[s:e], ignore_index, label_smoothing,
                                                   lse_square_scale)
            total += loss_rows.sum()
            if need_dx:
                dx[s:e] = _gemm.matmul_nn(dlogits, weight)           # (rows, H)
            if need_dw:
                _gemm.matmul_tn_acc_(dw, dlogits, xc)                # dw += dlogitsᵀ @ xc (fp32 accumulate)
            del logits, dlogits
        inv = 1.0 / n_valid
        ctx.save_for_backward(dx, dw, inv)
        ctx.wdtype = weight.dtype
        return total * inv

    @staticmethod
    def backward(ctx, gout):
        dx, dw, inv = ctx.saved_tensors
        s = gout * inv
        gx = (dx * s.to(dx.dtype)) if dx is not None else None
        gw = (dw * s).to(ctx.wdtype) if dw is not None else None
        return gx, gw, None, None, None, None, None


def default_chunk_rows(N: int, H: int, V: int, on_gpu: bool = False) -> int:
    """Rows per chunk.  The reference's rule makes the logits chunk about as large as the hidden states
    (``ceil(V / H)`` chunks, `lit_gpt/fused_linear_cross_entropy.py`): right when memory is the constraint, but every chunk
    is one more read-modify-write pass over the fp32 weight gradient ``[V, H]`` (2 GB for a 200 K vocabulary: 32 chunks of
    256 rows cost 130 GB of traffic for 8192 tokens).  On a GPU the chunk therefore grows until its logits reach a byte
    budget (``ARCHSCALE_B200_FLCE_CHUNK_MB``, default 2048 MiB of bf16 logits), never below the reference's size."""
    chunks = max(1, -(-V // max(H, 1)))
    chunks = min(chunks, 64)
    rows = -(-N // chunks)
    rows = max(256, ((rows + 255) // 256) * 256)
    if on_gpu:
        import os
        budget = int(float(os.environ.get("ARCHSCALE_B200_FLCE_CHUNK_MB", "2048")) * (1 << 20))
        by_budget = (budget // max(2 * V, 1)) // 256 * 256
        rows = max(rows, by_budget)
    return min(rows, N)


def fused_linear_cross_entropy(x: torch.Tensor, weight: torch.Tensor, target: torch.Tensor,
                               ignore_index: int = -100, label_smoothing: float = 0.0,
                               lse_square_scale: float = 0.0, chunk_rows: Optional[int] = None) -> torch.Tensor:
    """mean CE of ``(x @ weightᵀ)`` against ``target`` without materialising the logits.

    x: (..., H); weight: (V, H); target: (...) int64.
    """
    x2 = x.reshape(-1, x.shape[-1])
    t = target.reshape(-1)
    if chunk_rows is None:
        chunk_rows = default_chunk_rows(x2.shape[0], x2.shape[1], weight.shape[0], on_gpu=x2.is_cuda)
    return _FLCEFn.apply(x2, weight, t, ignore_index, label_smoothing, lse_square_scale, chunk_rows)


def fused_linear_cross_entropy_ref(x, weight, target, ignore_index: int = -100, label_smoothing: float = 0.0,
                                   lse_square_scale: float = 0.0) -> torch.Tensor:
    logits = x.reshape(-1, x.shape[-1]).float() @ weight.float().t()
    return cross_entropy_ref(logits, target.reshape(-1), ignore_index, label_smoothing, lse_square_scale)


class FusedLinearCrossEntropyLoss(torch.nn.Module):
    """Module form with the constructor arguments of the reference
    (`lit_gpt/fused_linear_cross_entropy.py:218-261`)."""

    def __init__(self, ignore_index: int = -100, label_smoothing: float = 0.0, lse_square_scale: float = 0.0,
                 reduction: str = "mean"):
        super().__init__()
        assert reduction == "mean"
        self.ignore_index, self.label_smoothing, self.lse_square_scale = ignore_index, label_smoothing, lse_square_scale

    def forward(self, hidden: torch.Tensor, weight: torch.Tensor, target: torch.Tensor) -> torch.Tensor:
        return fused_linear_cross_entropy(hidden, weight, target, self.ignore_index, self.label_smoothing,
                                          self.lse_square_scale)


class _CEFn(torch.autograd.Function):
    """Cross-entropy over materialised logits on the one-pass kernel (loss + dlogits in one read of the logits).  The
    gradient is computed in the forward pass into a copy of the logits — the caller's logits tensor is left intact,
    unlike the reference's in-place variant (`lit_gpt/fused_cross_entropy.py:29-150`, ``inplace_backward``)."""

    @staticmethod
    def forward(ctx, logits, target, ignore_index, label_smoothing, lse_square_scale, reduction):
        need = logits.requires_grad
        work = logits.detach().clone()       # the kernel overwrites its input with the gradient
        loss_rows, dlogits = _ce_chunk_fwd_bwd(work, target, ignore_index, label_smoothing, lse_square_scale)
        n_valid = (target != ignore_index).sum().clamp_min(1).to(torch.float32)
        ctx.reduction = reduction
        ctx.save_for_backward(dlogits if need else None, n_valid)
        if reduction == "none":
            return loss_rows
        return loss_rows.sum() / n_valid if reduction == "mean" else loss_rows.sum()

    @staticmethod
    def backward(ctx, gout):
        dlogits, n_valid = ctx.saved_tensors
        if dlogits is None:
            return (None,) * 6
        if ctx.reduction == "none":
            g = dlogits * gout.unsqueeze(1).to(dlogits.dtype)
        else:
            s = gout / n_valid if ctx.reduction == "mean" else gout
            g = dlogits * s.to(dlogits.dtype)
        return g, None, None, None, None, None


def cross_entropy(logits: torch.Tensor, target: torch.Tensor, ignore_index: int = -100, label_smoothing: float = 0.0,
                  lse_square_scale: float = 0.0, reduction: str = "mean") -> torch.Tensor:
    """CE of ``logits`` (N, V) against ``target`` (N,) on ``csrc/cross_entropy.cu`` (PyTorch formulas on CPU)."""
    return _CEFn.apply(logits.contiguous(), target, ignore_index, label_smoothing, lse_square_scale, reduction)


class FusedCrossEntropyLoss(torch.nn.Module):
    """Plain CE over materialised logits (`lit_gpt/fused_cross_entropy.py:336-415`)."""

    def __init__(self, ignore_index: int = -100, reduction: str = "mean", label_smoothing: float = 0.0,
                 lse_square_scale: float = 0.0, **_unused):
        super().__init__()
        self.ignore_index, self.reduction = ignore_index, reduction
        self.label_smoothing, self.lse_square_scale = label_smoothing, lse_square_scale

    def forward(self, logits: torch.Tensor, target: torch.Tensor) -> torch.Tensor:
        return cross_entropy(logits.reshape(-1, logits.shape[-1]), target.reshape(-1), self.ignore_index,
                             self.label_smoothing, self.lse_square_scale, self.reduction)
