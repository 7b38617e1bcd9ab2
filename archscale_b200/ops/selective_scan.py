"""Mamba-1 selective scan.

Behavioural reference: `lit_gpt/selective_scan_interface.py:102-168` (``selective_scan_ref``):
``h_t = exp(Δ_t·A)·h_{t-1} + Δ_t·B_t·u_t``, ``y_t = C_t·h_t + D·u_t``, optional ``·silu(z)``,
``Δ = softplus(Δ + bias)``; packed sequences reset ``h`` at every ``cu_seqlens`` boundary
(the varlen fork used at `lit_gpt/mamba_simple.py:84-88`).

CUDA path: ``csrc/selective_scan.cu`` — one thread per (batch, channel, state), 64-step tiles staged
through shared memory, state sums by warp shuffles; the backward recomputes each tile's states from
the per-tile checkpoints saved by the forward and runs the adjoint recurrence in reverse.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F

from . import backend


def selective_scan_ref(u, delta, A, B, C, D=None, z=None, delta_bias=None, delta_softplus: bool = False,
                       cu_seqlens: Optional[torch.Tensor] = None, return_last_state: bool = False):
    """u,delta,z:(B,Di,L)  A:(Di,N)  B,C:(B,N,L)  D:(Di,) → y:(B,Di,L)."""
    dtype_in = u.dtype
    u, delta = u.float(), delta.float()
    if delta_bias is not None:
        delta = delta + delta_bias.float().view(1, -1, 1)
    if delta_softplus:
        delta = F.softplus(delta)
    Bb, Di, L = u.shape
    N = A.shape[1]
    Bf, Cf = B.float(), C.float()
    dA = torch.exp(torch.einsum("bdl,dn->bdln", delta, A.float()))
    dBu = torch.einsum("bdl,bnl,bdl->bdln", delta, Bf, u)
    starts = set()
    if cu_seqlens is not None:
        starts = set(int(s) for s in cu_seqlens.tolist()[:-1])
    h = u.new_zeros(Bb, Di, N)
    ys = []
    for t in range(L):
        if t in starts:
            h = torch.zeros_like(h)
        h = dA[:, :, t] * h + dBu[:, :, t]
        ys.append(torch.einsum("bdn,bn->bd", h, Cf[:, :, t]))
    y = torch.stack(ys, dim=2)
    if D is not None:
        y = y + u * D.float().view(1, -1, 1)
    if z is not None:
        y = y * F.silu(z.float())
    y = y.to(dtype_in)
    return (y, h) if return_last_state else y


def _rows(t: torch.Tensor) -> torch.Tensor:
    """[B, L, C] with a dense last dimension and a uniform row stride (slices of a wider matrix qualify)."""
    if t.stride(2) == 1 and (t.size(0) == 1 or t.stride(0) == t.size(1) * t.stride(1)):
        return t
    return t.contiguous()


class _ScanFn(torch.autograd.Function):
    """Token-major kernel path: u, delta, z (B,L,Di); B, C (B,L,16); reset int32 (B·L,) or None."""

    @staticmethod
    def forward(ctx, u, delta, A, B, C, D, z, delta_bias, delta_softplus, reset):
        ext = backend.require_extension()
        u, delta, B, C = _rows(u), _rows(delta), _rows(B), _rows(C)
        z = _rows(z) if z is not None else None
        need_grad = any(t is not None and t.requires_grad for t in (u, delta, A, B, C, D, z, delta_bias))
        y, ckpt = ext.selective_scan_fwd(u, delta, A, B, C, D, z, delta_bias, delta_softplus, reset, need_grad)
        backend.count_launch()
        none = torch.empty(0)
        ctx.save_for_backward(u, delta, A, B, C, D, z if z is not None else none,
                              delta_bias if delta_bias is not None else none,
                              reset if reset is not None else none, ckpt if ckpt is not None else none)
        ctx.flags = (delta_softplus, z is not None, delta_bias is not None, reset is not None)
        return y

    @staticmethod
    def backward(ctx, dy):
        ext = backend.require_extension()
        u, delta, A, B, C, D, z, dbias, reset, ckpt = ctx.saved_tensors
        sp, has_z, has_b, has_r = ctx.flags
        du, ddelta, dz, dA, dB, dC, dD, ddb = ext.selective_scan_bwd(
            _rows(dy), u, delta, A, B, C, D, z if has_z else None, dbias if has_b else None, sp,
            reset if has_r else None, ckpt)
        backend.count_launch()
        return (du, ddelta, dA, dB.to(B.dtype), dC.to(C.dtype), dD, dz if has_z else None,
                ddb if has_b else None, None, None)


def _reset_flags(cu_seqlens: torch.Tensor, n_tokens: int) -> torch.Tensor:
    r = torch.zeros(n_tokens + 1, dtype=torch.int32, device=cu_seqlens.device)
    r[cu_seqlens.long()] = 1
    return r[:n_tokens].contiguous()


def selective_scan(u, delta, A, B, C, D=None, z=None, delta_bias=None, delta_softplus: bool = False,
                   cu_seqlens: Optional[torch.Tensor] = None, channel_last: bool = False):
    """``channel_last=False``: u,delta,z (B,Di,L), B,C (B,N,L) as in the reference interface;
    ``channel_last=True``: u,delta,z (B,L,Di), B,C (B,L,N) — the kernel's native layout.  Returns y in the layout of u."""
    if (backend.has("selective_scan_fwd") and u.dtype in (torch.bfloat16, torch.float32) and A.shape[1] == 16 and D is not None
            and B.dim() == 3 and u.shape[1 if not channel_last else 2] % 16 == 0
            and backend.use_cuda_kernel("selective_scan", u, delta, A, B, C)):
        tm = (lambda t: t) if channel_last else (lambda t: t.transpose(1, 2))
        ut = tm(u)
        reset = None if cu_seqlens is None else _reset_flags(cu_seqlens, ut.shape[0] * ut.shape[1])
        y = _ScanFn.apply(ut, tm(delta).to(u.dtype), A.float().contiguous(), tm(B).to(u.dtype), tm(C).to(u.dtype),
                          D.float().contiguous(), None if z is None else tm(z).to(u.dtype),
                          None if delta_bias is None else delta_bias.float().contiguous(), delta_softplus, reset)
        return tm(y)
    if channel_last:
        t = lambda v: None if v is None else v.transpose(1, 2)
        return _scan_chunked_torch(t(u), t(delta), A, t(B), t(C), D, t(z), delta_bias, delta_softplus,
                                   cu_seqlens).transpose(1, 2)
    return _scan_chunked_torch(u, delta, A, B, C, D, z, delta_bias, delta_softplus, cu_seqlens)


def _scan_chunked_torch(u, delta, A, B, C, D, z, delta_bias, delta_softplus, cu_seqlens):
    """Differentiable torch path (CPU backend).  Same math as the oracle, O(L) python loop over
    time is avoided with a log-space cumulative product inside chunks of 64 steps."""
    dtype_in = u.dtype
    uf, df = u.float(), delta.float()
    if delta_bias is not None:
        df = df + delta_bias.float().view(1, -1, 1)
    if delta_softplus:
        df = F.softplus(df)
    Bb, Di, L = uf.shape
    N = A.shape[1]
    Af = A.float()
    Bf, Cf = B.float(), C.float()
    reset = torch.zeros(L, dtype=torch.bool, device=u.device)
    if cu_seqlens is not None:
        reset[cu_seqlens[:-1].long()] = True
    T = 64
    h = uf.new_zeros(Bb, Di, N)
    outs = []
    for s in range(0, L, T):
        e = min(s + T, L)
        d = df[:, :, s:e]                                            # B Di t
        la = torch.einsum("bdt,dn->bdtn", d, Af)                     # log decay per step (<= 0)
        r = reset[s:e]
        if r.any():
            la = la.masked_fill(r.view(1, 1, -1, 1), float("-inf"))
        cs = torch.cumsum(la.masked_fill(torch.isinf(la), 0.0), dim=2)
        # number of resets up to and including step t: contributions from before a reset are dropped
        rc = torch.cumsum(r.to(torch.int32), dim=0)                  # t
        x = torch.einsum("bdt,bnt,bdt->bdtn", d, Bf[:, :, s:e], uf[:, :, s:e])
        # h_t = Σ_{s<=t, same segment} exp(cs_t - cs_s) x_s  + exp(cs_t) h_in (if no reset yet)
        tt = e - s
        diff = cs.unsqueeze(3) - cs.unsqueeze(2)                     # B Di t s N
        same = (rc.view(-1, 1) == rc.view(1, -1)) & (torch.arange(tt, device=u.device).view(-1, 1) >=
                                                     torch.arange(tt, device=u.device).view(1, -1))
        w = torch.exp(diff.masked_fill(~same.view(1, 1, tt, tt, 1), float("-inf")))
        hs = torch.einsum("bdtsn,bdsn->bdtn", w, x)
        carry = torch.exp(cs) * (rc == 0).view(1, 1, -1, 1)
        hs = hs + carry * h.unsqueeze(2)
        outs.append(torch.einsum("bdtn,bnt->bdt", hs, Cf[:, :, s:e]))
        h = hs[:, :, -1]
    y = torch.cat(outs, dim=2)
    if D is not None:
        y = y + uf * D.float().view(1, -1, 1)
    if z is not None:
        y = y * F.silu(z.float())
    return y.to(dtype_in)
