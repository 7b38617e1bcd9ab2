"""Gated delta rule (Gated DeltaNet) sequence mixer core.

Behavioural reference: the ``chunk_gated_delta_rule(q, k, v, g, beta, use_qk_l2norm_in_kernel=True)``
call at `lit_gpt/gated_deltanet.py:315-326`.  Per head, with state ``S ∈ R^{Dk×Dv}``:

    S_t = exp(g_t)·S_{t-1} + β_t · k_t ⊗ (v_t − (exp(g_t)·S_{t-1})ᵀ k_t)
    o_t = (q_t·scale)ᵀ S_t

q, k are L2-normalised over the head dim first; ``g ≤ 0`` is a log-decay; ``β`` may reach 2
(negative eigenvalues).  Packed sequences reset ``S`` at ``cu_seqlens`` boundaries.

Two PyTorch implementations: :func:`gated_delta_rule_recurrent_ref` (step-by-step oracle) and
:func:`gated_delta_rule_chunk` (chunk-of-64 WY form, differentiable, all matmuls — the shape
the CUDA kernel ``csrc/gdn_chunk.cu`` follows).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F

from . import backend


def _l2norm(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    return x * torch.rsqrt(x.pow(2).sum(dim=-1, keepdim=True) + eps)


def gated_delta_rule_recurrent_ref(q, k, v, g, beta, scale: Optional[float] = None, l2norm: bool = True,
                                   cu_seqlens: Optional[torch.Tensor] = None):
    """q,k:(B,T,H,Dk) v:(B,T,H,Dv) g,beta:(B,T,H) → o:(B,T,H,Dv) (fp32 math)."""
    dtype = v.dtype
    q, k, v, g, beta = (t.float() for t in (q, k, v, g, beta))
    if l2norm:
        q, k = _l2norm(q), _l2norm(k)
    B, T, H, Dk = q.shape
    Dv = v.shape[-1]
    scale = Dk ** -0.5 if scale is None else scale
    starts = set() if cu_seqlens is None else set(int(s) for s in cu_seqlens.tolist()[:-1])
    S = q.new_zeros(B, H, Dk, Dv)
    out = []
    for t in range(T):
        if t in starts:
            S = torch.zeros_like(S)
        S = S * torch.exp(g[:, t]).unsqueeze(-1).unsqueeze(-1)
        kt, vt, bt = k[:, t], v[:, t], beta[:, t].unsqueeze(-1)
        pred = torch.einsum("bhkv,bhk->bhv", S, kt)
        S = S + torch.einsum("bhk,bhv->bhkv", kt, (vt - pred) * bt)
        out.append(torch.einsum("bhkv,bhk->bhv", S, q[:, t] * scale))
    return torch.stack(out, dim=1).to(dtype)


def gated_delta_rule_chunk(q, k, v, g, beta, scale: Optional[float] = None, l2norm: bool = True,
                           cu_seqlens: Optional[torch.Tensor] = None, chunk: int = 64):
    """Chunked WY formulation.  Equivalent to the recurrent oracle; differentiable."""
    dtype = v.dtype
    B, T, H, Dk = q.shape
    Dv = v.shape[-1]
    if cu_seqlens is not None:
        # documents are processed one by one so that no chunk spans a boundary
        assert B == 1
        outs = []
        cl = cu_seqlens.tolist()
        for s, e in zip(cl[:-1], cl[1:]):
            if e > s:
                outs.append(gated_delta_rule_chunk(q[:, s:e], k[:, s:e], v[:, s:e], g[:, s:e], beta[:, s:e],
                                                   scale, l2norm, None, chunk))
        return torch.cat(outs, dim=1)
    q, k, v, g, beta = (t.float() for t in (q, k, v, g, beta))
    if l2norm:
        q, k = _l2norm(q), _l2norm(k)
    scale = Dk ** -0.5 if scale is None else scale
    pad = (-T) % chunk
    if pad:
        q, k, v = (F.pad(t, (0, 0, 0, 0, 0, pad)) for t in (q, k, v))
        g, beta = (F.pad(t, (0, 0, 0, pad)) for t in (g, beta))
    Tp = T + pad
    nC = Tp // chunk
    # (B,H,nC,c,·)
    r = lambda t: t.permute(0, 2, 1, 3).reshape(B, H, nC, chunk, t.shape[-1])
    q, k, v = r(q) * scale, r(k), r(v)
    g = g.permute(0, 2, 1).reshape(B, H, nC, chunk)
    beta = beta.permute(0, 2, 1).reshape(B, H, nC, chunk)
    gc = torch.cumsum(g, dim=-1)                                         # inclusive log-decay inside the chunk
    kb = k * beta.unsqueeze(-1)
    vb = v * beta.unsqueeze(-1)
    dec = torch.exp(gc.unsqueeze(-1) - gc.unsqueeze(-2))                 # [i,j] = exp(gc_i - gc_j)
    strict = torch.tril(torch.ones(chunk, chunk, device=q.device, dtype=torch.bool), -1)
    incl = torch.tril(torch.ones(chunk, chunk, device=q.device, dtype=torch.bool), 0)
    A = torch.einsum("bhnik,bhnjk->bhnij", kb, k) * dec
    A = A.masked_fill(~strict, 0.0)
    eye = torch.eye(chunk, device=q.device, dtype=q.dtype)
    # (I + A) is unit lower-triangular → solve for W, U:  (I+A) U = β v ; (I+A) W = β k·exp(gc)
    Tm = torch.linalg.solve_triangular(eye + A, eye.expand_as(A), upper=False, unitriangular=True)
    u = Tm @ vb
    w = Tm @ (kb * torch.exp(gc).unsqueeze(-1))
    S = q.new_zeros(B, H, Dk, Dv)
    qk = (torch.einsum("bhnik,bhnjk->bhnij", q, k) * dec).masked_fill(~incl, 0.0)
    outs = []
    for n in range(nC):
        v_new = u[:, :, n] - w[:, :, n] @ S                              # c × Dv
        o_inter = (q[:, :, n] * torch.exp(gc[:, :, n]).unsqueeze(-1)) @ S
        outs.append(o_inter + qk[:, :, n] @ v_new)
        g_last = gc[:, :, n, -1]
        kdec = k[:, :, n] * torch.exp(g_last.unsqueeze(-1) - gc[:, :, n]).unsqueeze(-1)
        S = S * torch.exp(g_last).unsqueeze(-1).unsqueeze(-1) + kdec.transpose(-1, -2) @ v_new
    o = torch.stack(outs, dim=2).reshape(B, H, Tp, Dv).permute(0, 2, 1, 3)[:, :T]
    return o.to(dtype)


def gated_delta_rule(q, k, v, g, beta, scale: Optional[float] = None, l2norm: bool = True,
                     cu_seqlens: Optional[torch.Tensor] = None):
    return gated_delta_rule_chunk(q, k, v, g, beta, scale, l2norm, cu_seqlens)
