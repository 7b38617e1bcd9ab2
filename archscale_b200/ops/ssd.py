"""Mamba-2 state-space-duality (SSD) scan.

Behavioural reference: the ``mamba_chunk_scan_combined`` call at `lit_gpt/mamba2.py:289-305`:
per head ``h`` with scalar decay ``A_h < 0``:

    S_t = exp(dt_t·A_h)·S_{t-1} + dt_t · x_t ⊗ B_t ;   y_t = S_t C_t + D_h·x_t

x:(B,L,H,P) dt:(B,L,H) (after softplus+bias) A:(H,) B,C:(B,L,G,N) D:(H,).  ``seq_idx`` resets
the state at document boundaries.  Chunked (256) matmul form below is differentiable.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F


def ssd_scan_ref(x, dt, A, B, C, D=None, seq_idx: Optional[torch.Tensor] = None):
    dtype = x.dtype
    x, dt, B, C = x.float(), dt.float(), B.float(), C.float()
    Bb, L, H, P = x.shape
    G, N = B.shape[2], B.shape[3]
    Bh = B.repeat_interleave(H // G, dim=2)
    Ch = C.repeat_interleave(H // G, dim=2)
    S = x.new_zeros(Bb, H, P, N)
    ys = []
    for t in range(L):
        if seq_idx is not None and t > 0:
            keep = (seq_idx[:, t] == seq_idx[:, t - 1]).view(Bb, 1, 1, 1).float()
            S = S * keep
        dA = torch.exp(dt[:, t] * A.float().view(1, H))
        S = S * dA.view(Bb, H, 1, 1) + torch.einsum("bh,bhp,bhn->bhpn", dt[:, t], x[:, t], Bh[:, t])
        ys.append(torch.einsum("bhpn,bhn->bhp", S, Ch[:, t]))
    y = torch.stack(ys, dim=1)
    if D is not None:
        y = y + x * D.float().view(1, 1, H, 1)
    return y.to(dtype)


def ssd_scan(x, dt, A, B, C, D=None, seq_idx: Optional[torch.Tensor] = None, chunk: int = 128):
    """Chunked quadratic-within-chunk / recurrent-across-chunk form (differentiable)."""
    dtype = x.dtype
    x, dt, B, C = x.float(), dt.float(), B.float(), C.float()
    Bb, L, H, P = x.shape
    G, N = B.shape[2], B.shape[3]
    Bh = B.repeat_interleave(H // G, dim=2)
    Ch = C.repeat_interleave(H // G, dim=2)
    la = dt * A.float().view(1, 1, H)                                   # log decay per step
    if seq_idx is not None:
        brk = torch.zeros(Bb, L, dtype=torch.bool, device=x.device)
        brk[:, 1:] = seq_idx[:, 1:] != seq_idx[:, :-1]
    else:
        brk = torch.zeros(Bb, L, dtype=torch.bool, device=x.device)
    S = x.new_zeros(Bb, H, P, N)
    outs = []
    for s in range(0, L, chunk):
        e = min(s + chunk, L)
        t = e - s
        l = la[:, s:e].permute(0, 2, 1)                                 # B H t
        cs = torch.cumsum(l, dim=-1)
        bc = torch.cumsum(brk[:, s:e].to(torch.int32), dim=-1)          # B t (breaks so far, inclusive)
        same = (bc.unsqueeze(-1) == bc.unsqueeze(-2)) & torch.tril(
            torch.ones(t, t, dtype=torch.bool, device=x.device)).unsqueeze(0)
        w = torch.exp((cs.unsqueeze(-1) - cs.unsqueeze(-2)).masked_fill(~same.unsqueeze(1), float("-inf")))
        xb = x[:, s:e] * dt[:, s:e].unsqueeze(-1)                       # B t H P
        cb = torch.einsum("bihn,bjhn->bhij", Ch[:, s:e], Bh[:, s:e]) * w
        y = torch.einsum("bhij,bjhp->bihp", cb, xb)
        carry = torch.exp(cs) * (bc == 0).unsqueeze(1)                  # B H t
        y = y + torch.einsum("bhpn,bihn,bhi->bihp", S, Ch[:, s:e], carry)
        outs.append(y)
        # state at the end of the chunk
        last_same = same[:, -1]                                         # B t : steps in the last segment
        wl = torch.exp((cs[:, :, -1:] - cs).masked_fill(~last_same.unsqueeze(1), float("-inf")))
        S = S * carry[:, :, -1].view(Bb, H, 1, 1) + torch.einsum("bhj,bjhp,bjhn->bhpn", wl, xb, Bh[:, s:e])
    y = torch.cat(outs, dim=1)
    if D is not None:
        y = y + x * D.float().view(1, 1, H, 1)
    return y.to(dtype)
