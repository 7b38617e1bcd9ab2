"""Mamba-2 state-space-duality (SSD) scan.

Behavioural reference: the ``mamba_chunk_scan_combined`` call at `lit_gpt/mamba2.py:289-305`:
per head ``h`` with scalar decay ``A_h < 0``:

    S_t = exp(dt_t·A_h)·S_{t-1} + dt_t · x_t ⊗ B_t ;   y_t = S_t C_t + D_h·x_t

x:(B,L,H,P) dt:(B,L,H) (after softplus+bias) A:(H,) B,C:(B,L,G,N) D:(H,).  ``seq_idx`` resets
the state at document boundaries.  The chunked matmul form below is differentiable.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F

from . import backend


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


def chunk_state_scan_ref(add: torch.Tensor, keep: torch.Tensor) -> torch.Tensor:
    """``S_in[:, 0] = 0, S_in[:, n+1] = keep[:, n]·S_in[:, n] + add[:, n]`` — add (B,nC,H,P,N), keep (B,nC,H)."""
    Bb, nC, H, P, N = add.shape
    S = add.new_zeros(Bb, H, P, N)
    states = []
    for n in range(nC):                                                                  # the only sequential part
        states.append(S)
        S = S * keep[:, n].view(Bb, H, 1, 1) + add[:, n]
    return torch.stack(states, dim=1)


class _StateScanFn(torch.autograd.Function):
    """The recurrence over chunks as one kernel each way (``csrc/ssd_scan.cu``)."""

    @staticmethod
    def forward(ctx, add, keep):
        add, keep = add.contiguous(), keep.contiguous()
        s_in = backend.require_extension().ssd_state_fwd(add, keep)
        backend.count_launch()
        ctx.save_for_backward(s_in, keep)
        return s_in

    @staticmethod
    def backward(ctx, d_s_in):
        s_in, keep = ctx.saved_tensors
        d_add, d_keep = backend.require_extension().ssd_state_bwd(d_s_in.contiguous(), s_in, keep)
        backend.count_launch(2)
        return d_add, d_keep


class _IntraChunkFn(torch.autograd.Function):
    """``y[i] = Σ_{j ≤ i, same document} (C_i·B_j) · exp(cs_i − cs_j) · dt_j · x_j`` inside every chunk, on
    ``csrc/ssd_intra.cu``: the per-head 64×64 weights never reach memory.  x (B,Lp,H,P), dt (B,Lp,H), cs (B,nC,H,64),
    cb (B,nC,G,64,64), bc (B,nC,64) int32 or None → y (B,Lp,H,P) fp32."""

    @staticmethod
    def forward(ctx, x, dt, cs, cb, bc):
        x, dt, cs, cb = x.contiguous(), dt.contiguous(), cs.contiguous(), cb.contiguous()
        y = backend.require_extension().ssd_intra_fwd(x, dt, cs, cb, bc)
        backend.count_launch()
        ctx.save_for_backward(x, dt, cs, cb, bc)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, dt, cs, cb, bc = ctx.saved_tensors
        dx, ddt, dcs, dcb = backend.require_extension().ssd_intra_bwd(x, dt, cs, cb, bc, dy.float().contiguous())
        backend.count_launch()
        Bb, Lp, H, _ = x.shape
        return dx.to(x.dtype), ddt.permute(0, 1, 3, 2).reshape(Bb, Lp, H), dcs, dcb, None


def _intra_kernel_ok(x: torch.Tensor, c: int) -> bool:
    return (x.is_cuda and c == 64 and x.shape[-1] % 64 == 0 and x.dtype in (torch.float32, torch.bfloat16)
            and backend.has("ssd_intra_fwd") and backend.use_cuda_kernel("ssd", x))


def chunk_state_scan(add: torch.Tensor, keep: torch.Tensor) -> torch.Tensor:
    if (add.is_cuda and add.dtype == torch.float32 and keep.dtype == torch.float32 and (add.shape[3] * add.shape[4]) % 1024 == 0
            and backend.has("ssd_state_fwd") and backend.use_cuda_kernel("ssd", add)):
        return _StateScanFn.apply(add, keep)
    return chunk_state_scan_ref(add, keep)


def ssd_scan(x, dt, A, B, C, D=None, seq_idx: Optional[torch.Tensor] = None, chunk: int = 64):
    """Chunked form, vectorised over the chunks: the quadratic work inside a chunk and the chunk summaries are batched
    matmuls over all chunks at once; only the (B,H,P,N) state is carried from chunk to chunk in a short loop of
    element-wise updates.  Differentiable; equals :func:`ssd_scan_ref`."""
    dtype = x.dtype
    x, dt, B, C = x.float(), dt.float(), B.float(), C.float()
    Bb, L, H, P = x.shape
    G, N = B.shape[2], B.shape[3]
    pad = (-L) % chunk
    if seq_idx is not None:
        brk = torch.zeros(Bb, L, dtype=torch.bool, device=x.device)
        brk[:, 1:] = seq_idx[:, 1:] != seq_idx[:, :-1]
    else:
        brk = None
    if pad:
        # padded steps have dt = 0: they neither decay nor write the state, and their outputs are cut off
        x, B, C = (F.pad(t, (0, 0, 0, 0, 0, pad)) for t in (x, B, C))
        dt = F.pad(dt, (0, 0, 0, pad))
        if brk is not None:
            brk = F.pad(brk, (0, pad))
    Lp = L + pad
    nC, c = Lp // chunk, chunk
    xb_cache = []

    def xb():                                          # dt·x in chunk layout, formed only by the paths that read it
        if not xb_cache:
            xb_cache.append((x * dt.unsqueeze(-1)).view(Bb, nC, c, H, P))
        return xb_cache[0]

    la = (dt * A.float().view(1, 1, H)).view(Bb, nC, c, H).permute(0, 1, 3, 2)          # (B,nC,H,c) log decay per step
    cs = torch.cumsum(la, dim=-1)                                                        # inclusive, inside the chunk
    tril = torch.tril(torch.ones(c, c, dtype=torch.bool, device=x.device))
    if brk is not None:
        bc = torch.cumsum(brk.view(Bb, nC, c).to(torch.int32), dim=-1)                   # breaks so far inside the chunk
        same = (bc.unsqueeze(-1) == bc.unsqueeze(-2)) & tril                              # (B,nC,c,c): j reaches i
        first = (bc == 0)                                                                 # still the segment entering the chunk
        last_same = same[:, :, -1]                                                        # (B,nC,c): steps of the last segment
    else:
        same = tril.view(1, 1, c, c)
        first = last_same = None
    # inside a chunk: y_i = Σ_{j≤i} (C_i·B_j) · exp(cs_i − cs_j) · dt_j x_j
    Bh = B.view(Bb, nC, c, G, N)
    Ch = C.view(Bb, nC, c, G, N)
    cb = torch.einsum("bnigk,bnjgk->bngij", Ch, Bh)                                      # (B,nC,G,c,c)
    rep = H // G
    if _intra_kernel_ok(x, c):
        y = _IntraChunkFn.apply(x, dt, cs, cb, bc.to(torch.int32).contiguous() if brk is not None else None)
        y = y.view(Bb, nC, c, H, P)
    else:
        dec = cs.unsqueeze(-1) - cs.unsqueeze(-2)                                        # (B,nC,H,c,c)
        w = torch.exp(dec.masked_fill(~same.unsqueeze(2), float("-inf")))
        wg = w.view(Bb, nC, G, rep, c, c) * cb.unsqueeze(3)
        y = torch.einsum("bngrij,bnjgrp->bnigrp", wg, xb().view(Bb, nC, c, G, rep, P)).reshape(Bb, nC, c, H, P)
    # chunk summaries: what each chunk adds to the state by its end, and how much of the entering state survives it
    wl = torch.exp(cs[..., -1:] - cs)                                                    # (B,nC,H,c)
    carry = torch.exp(cs)                                                                # decay from the chunk start to step i
    if brk is not None:
        wl = wl * last_same.unsqueeze(2)
        carry = carry * first.unsqueeze(2)
    keep = carry[..., -1]                                                                # (B,nC,H)
    if G == 1:
        # one group: inside a chunk the token-major layout (c, H·P) is already what a batched matmul over the chunks wants,
        # so both products run without operand permutes or per-head copies of B / C
        BN = Bb * nC
        xw = (x.view(Bb, nC, c, H, P) * (dt.view(Bb, nC, c, H) * wl.permute(0, 1, 3, 2)).unsqueeze(-1)).view(BN, c, H * P)
        add = torch.bmm(xw.transpose(1, 2), Bh.reshape(BN, c, N)).view(Bb, nC, H, P, N)
        S_in = chunk_state_scan(add, keep)                                               # state entering each chunk
        y2 = torch.bmm(Ch.reshape(BN, c, N), S_in.view(BN, H * P, N).transpose(1, 2)).view(Bb, nC, c, H, P)
        y = torch.addcmul(y, y2, carry.permute(0, 1, 3, 2).unsqueeze(-1))
    else:
        add = torch.einsum("bngrj,bnjgrp,bnjgk->bngrpk", wl.view(Bb, nC, G, rep, c), xb().view(Bb, nC, c, G, rep, P), Bh)
        add = add.reshape(Bb, nC, H, P, N)
        S_in = chunk_state_scan(add, keep)                                               # state entering each chunk
        y = y + torch.einsum("bngrpk,bnigk,bngri->bnigrp", S_in.view(Bb, nC, G, rep, P, N), Ch,
                             carry.view(Bb, nC, G, rep, c)).reshape(Bb, nC, c, H, P)
    y = y.reshape(Bb, Lp, H, P)[:, :L]
    if D is not None:
        y = y + x[:, :L] * D.float().view(1, 1, H, 1)
    return y.to(dtype)
