"""Gated delta rule (Gated DeltaNet) sequence mixer core.

Behavioural reference: the ``chunk_gated_delta_rule(q, k, v, g, beta, use_qk_l2norm_in_kernel=True)``
call at `lit_gpt/gated_deltanet.py:315-326`.  Per head, with state ``S ∈ R^{Dk×Dv}``:

    S_t = exp(g_t)·S_{t-1} + β_t · k_t ⊗ (v_t − (exp(g_t)·S_{t-1})ᵀ k_t)
    o_t = (q_t·scale)ᵀ S_t

q, k are L2-normalised over the head dim first; ``g ≤ 0`` is a log-decay; ``β`` may reach 2
(negative eigenvalues).  Packed sequences reset ``S`` at ``cu_seqlens`` boundaries.

Implementations: :func:`gated_delta_rule_recurrent_ref` (step-by-step oracle) and
:func:`gated_delta_rule_chunk` (chunk-of-64 WY form, differentiable).  In the chunk form everything is a batched
matmul over independent chunks except one recurrence over the chunks of a sequence; on a GPU that recurrence runs
in the tcgen05 kernel ``csrc/gdn_chunk.cu`` (forward and, over the chunks in reverse, backward) and the
chunk-parallel products around it are batched library matmuls.
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


def _chunk_core_ref(w, u, kd, qg, qk, a):
    """The recurrence over chunks in plain PyTorch.  w, kd, qg: (BH,nC,c,Dk); u: (BH,nC,c,Dv); qk: (BH,nC,c,c);
    a: (BH,nC) → o: (BH,nC,c,Dv).  With S the (Dk×Dv) state at the chunk start:
    ``v = u − w·S``, ``o = qg·S + qk·v``, ``S ← a·S + kdᵀ·v``."""
    BH, nC, _, Dk = w.shape
    S = w.new_zeros(BH, Dk, u.shape[-1])
    outs = []
    for n in range(nC):
        v_new = u[:, n] - w[:, n] @ S
        outs.append(qg[:, n] @ S + qk[:, n] @ v_new)
        S = S * a[:, n, None, None] + kd[:, n].transpose(-1, -2) @ v_new
    return torch.stack(outs, dim=1)


def _gdn_state_ref(a_op, c_add, bm_op, e_op, f_op, decay, reverse: bool, sgn_p: float, sgn_v: float):
    """What one launch of the ``gdn_state`` kernel computes, in PyTorch (operand dtype kept, fp32 state).  With the
    transposed state X (Dv×Dk), per chunk n: ``P = X·Aᵀ``, ``V = C + sgn_p·Pᵀ``, ``X ← a_n·X + sgn_v·Vᵀ·Bm (+ Eᵀ·F)``;
    returns V, the state each chunk saw, and the final state."""
    BH, Tp, Dk = a_op.shape
    Dv, nC = c_add.shape[-1], Tp // 64
    ch = lambda t: t.reshape(BH, nC, 64, t.shape[-1]).float()
    A, C, Bm = ch(a_op), ch(c_add), ch(bm_op)
    X = A.new_zeros(BH, Dv, Dk)
    v_out, x_all = torch.empty_like(C), A.new_empty(BH, nC, Dv, Dk)
    for s in range(nC):
        n = nC - 1 - s if reverse else s
        Xr = X.to(a_op.dtype).float()
        x_all[:, n] = Xr
        V = (C[:, n] + sgn_p * (Xr @ A[:, n].transpose(-1, -2)).transpose(-1, -2)).to(a_op.dtype).float()
        v_out[:, n] = V
        X = X * decay[:, n, None, None].float() + sgn_v * (V.transpose(-1, -2) @ Bm[:, n])
        if e_op is not None:
            X = X + ch(e_op)[:, n].transpose(-1, -2) @ ch(f_op)[:, n]
    return v_out.reshape(BH, Tp, Dv).to(a_op.dtype), x_all.to(a_op.dtype), X


def _gdn_state(a_op, c_add, bm_op, e_op, f_op, decay, reverse, sgn_p, sgn_v):
    if a_op.is_cuda:
        out = backend.require_extension().gdn_state(a_op, c_add, bm_op, e_op, f_op, decay, reverse, sgn_p, sgn_v)
        backend.count_launch()
        return out
    return _gdn_state_ref(a_op, c_add, bm_op, e_op, f_op, decay, reverse, sgn_p, sgn_v)


class _ChunkCoreFn(torch.autograd.Function):
    """Same contract as :func:`_chunk_core_ref`; the recurrence runs in ``gdn_state`` (bf16 operands, fp32 state)."""

    @staticmethod
    def forward(ctx, w, u, kd, qg, qk, a):
        BH, nC, c, Dk = w.shape
        Dv = u.shape[-1]
        bf = torch.bfloat16 if w.is_cuda else w.dtype          # the kernel takes bf16 operands
        wb, ub, kdb, qgb = (t.to(bf).reshape(BH, nC * c, -1).contiguous() for t in (w, u, kd, qg))
        qkb, af = qk.to(bf).contiguous(), a.float().contiguous()
        v, s_all, _ = _gdn_state(wb, ub, kdb, None, None, af, False, -1.0, 1.0)
        o = qgb.view(BH, nC, c, Dk) @ s_all.transpose(-1, -2) + qkb @ v.view(BH, nC, c, Dv)
        ctx.save_for_backward(wb, ub, kdb, qgb, qkb, af)
        ctx.dtypes = (w.dtype, u.dtype, kd.dtype, qg.dtype, qk.dtype, a.dtype)
        return o.to(u.dtype)

    @staticmethod
    def backward(ctx, do):
        wb, ub, kdb, qgb, qkb, af = ctx.saved_tensors
        BH, nC, c, _ = qkb.shape
        Dk, Dv = wb.shape[-1], ub.shape[-1]
        # the states are not kept between the passes: the forward recurrence runs again
        v, s_all, _ = _gdn_state(wb, ub, kdb, None, None, af, False, -1.0, 1.0)
        dob = do.to(wb.dtype).contiguous()                                     # (BH,nC,c,Dv)
        g = (qkb.transpose(-1, -2) @ dob).reshape(BH, nC * c, Dv)              # ∂L/∂v through o = qk·v
        dv, ds_all, _ = _gdn_state(kdb, g, wb, dob.view(BH, nC * c, Dv), qgb, af, True, 1.0, -1.0)
        v4, dv4 = v.view(BH, nC, c, Dv), dv.view(BH, nC, c, Dv)
        dqg = dob @ s_all                                                      # s_all: (BH,nC,Dv,Dk)
        dqk = dob @ v4.transpose(-1, -2)
        dw = -(dv4 @ s_all)
        dkd = v4 @ ds_all                                                      # ds_all[n] = ∂L/∂S after chunk n
        da = (s_all * ds_all).sum((-1, -2), dtype=torch.float32)
        dt = ctx.dtypes
        return dw.to(dt[0]), dv4.to(dt[1]), dkd.to(dt[2]), dqg.to(dt[3]), dqk.to(dt[4]), da.to(dt[5])


class _TriInverseFn(torch.autograd.Function):
    """``(I + A)⁻¹`` for strictly lower-triangular 64×64 blocks on the substitution kernel (``csrc/tri_inverse.cu``);
    backward from ``dA = −Tᵀ · dT · Tᵀ`` (strictly lower part)."""

    @staticmethod
    def forward(ctx, A):
        T = backend.require_extension().tri_inverse64(A.contiguous())
        backend.count_launch()
        ctx.save_for_backward(T)
        return T

    @staticmethod
    def backward(ctx, dT):
        (T,) = ctx.saved_tensors
        Tt = T.transpose(-1, -2)
        return (-(Tt @ dT @ Tt)).tril(-1)


def unit_lower_inverse(A: torch.Tensor) -> torch.Tensor:
    """``(I + A)⁻¹`` for strictly lower-triangular ``A (…, c, c)``."""
    c = A.shape[-1]
    if (A.is_cuda and c == 64 and A.dtype == torch.float32 and backend.has("tri_inverse64")
            and backend.use_cuda_kernel("gated_delta_rule", A)):
        return _TriInverseFn.apply(A)
    eye = torch.eye(c, device=A.device, dtype=A.dtype)
    return torch.linalg.solve_triangular(eye + A, eye.expand_as(A), upper=False, unitriangular=True)


def _chunk_core(w, u, kd, qg, qk, a):
    Dk, Dv = w.shape[-1], u.shape[-1]
    if (w.is_cuda and w.shape[2] == 64 and Dk in (128, 256) and Dv % 128 == 0 and backend.has("gdn_state")
            and backend.use_cuda_kernel("gated_delta_rule", w, u)):
        return _ChunkCoreFn.apply(w, u, kd, qg, qk, a)
    return _chunk_core_ref(w, u, kd, qg, qk, a)


class _PrepareFn(torch.autograd.Function):
    """(q, k, v token-major bf16; gc chunk-major fp32) → (qn, kn, vc, kd, qg) chunk-major bf16 on ``csrc/gdn_prepare.cu``:
    l2-normalisation, the softmax scale, the two decay factors and the layout change in one pass each way."""

    @staticmethod
    def forward(ctx, q, k, v, gc, scale, eps):
        q, k, v, gc = q.contiguous(), k.contiguous(), v.contiguous(), gc.contiguous()
        outs = backend.require_extension().gdn_prepare_fwd(q, k, v, gc, scale, eps)
        backend.count_launch()
        ctx.save_for_backward(q, k, v, gc)
        ctx.consts = (scale, eps)
        return tuple(outs)

    @staticmethod
    def backward(ctx, dqn, dkn, dvc, dkd, dqg):
        q, k, v, gc = ctx.saved_tensors
        scale, eps = ctx.consts
        z = lambda t, ref_d: (t if t is not None else torch.zeros(gc.shape[0], gc.shape[1], ref_d, dtype=q.dtype, device=q.device)).contiguous()
        Dk, Dv = q.shape[-1], v.shape[-1]
        dq, dk, dv, a_row, s_row = backend.require_extension().gdn_prepare_bwd(
            q, k, v, gc, z(dqn, Dk), z(dkn, Dk), z(dvc, Dv), z(dkd, Dk), z(dqg, Dk), scale, eps)
        backend.count_launch()
        # gc enters through qg = qn·exp(gc) and kd = kn·exp(gl − gc), gl = gc at the chunk's last token
        s_c = s_row.view(gc.shape[0], -1, 64)
        dgc = (a_row.view_as(s_c) - s_c).clone()
        dgc[..., -1] += s_c.sum(-1)
        return dq, dk, dv, dgc.view_as(gc), None, None


class _BmmNTf32(torch.autograd.Function):
    """``a @ bᵀ`` for bf16 operands with an fp32 result (the 64×64 Gram blocks feed a triangular inverse); gradients in bf16."""

    @staticmethod
    def forward(ctx, a, b):
        ctx.save_for_backward(a, b)
        try:
            return torch.bmm(a.flatten(0, -3), b.flatten(0, -3).transpose(-1, -2), out_dtype=torch.float32).view(*a.shape[:-1], b.shape[-2])
        except (TypeError, RuntimeError):
            return a.float() @ b.float().transpose(-1, -2)

    @staticmethod
    def backward(ctx, g):
        a, b = ctx.saved_tensors
        gb = g.to(a.dtype)
        return gb @ b, gb.transpose(-1, -2) @ a


def _prepare_kernel_ok(q, k, v, chunk: int, l2norm: bool) -> bool:
    Dk, Dv = q.shape[-1], v.shape[-1]
    return (q.is_cuda and l2norm and chunk == 64 and q.dtype == torch.bfloat16 and k.dtype == torch.bfloat16 and v.dtype == torch.bfloat16
            and (Dk, Dv) in ((128, 128), (128, 256), (256, 256), (256, 512)) and backend.has("gdn_prepare_fwd")
            and backend.has("gdn_state") and backend.use_cuda_kernel("gated_delta_rule", q, k, v))


def _chunk_fused_prepare(q, k, v, g, beta, scale: float, eps: float = 1e-6):
    """The chunked form with the row-wise work on the prepare kernels and bf16 operands for every product; the 64×64
    pieces (decay matrix, masks, triangular inverse, its column scalings) stay small fp32 PyTorch ops."""
    B, T, H, Dk = q.shape
    Dv = v.shape[-1]
    c = 64
    Tp = -(-T // c) * c
    nC = Tp // c
    g = g.float().permute(0, 2, 1).reshape(B * H, T)
    beta = beta.float().permute(0, 2, 1).reshape(B * H, T)
    if Tp != T:
        g, beta = F.pad(g, (0, Tp - T)), F.pad(beta, (0, Tp - T))
    gc = torch.cumsum(g.view(B * H, nC, c), dim=-1)                      # inclusive log-decay inside the chunk
    beta = beta.view(B * H, nC, c)
    qn, kn, vc, kd, qg = _PrepareFn.apply(q, k, v, gc.view(B * H, Tp), float(scale), eps)
    r4 = lambda t: t.view(B * H, nC, c, t.shape[-1])
    qn, kn, vc, kd, qg = r4(qn), r4(kn), r4(vc), r4(kd), r4(qg)
    dec = torch.exp(gc.unsqueeze(-1) - gc.unsqueeze(-2))                 # [i, j] = exp(gc_i − gc_j)
    strict = torch.tril(torch.ones(c, c, device=q.device, dtype=torch.bool), -1)
    incl = torch.tril(torch.ones(c, c, device=q.device, dtype=torch.bool), 0)
    A = (_BmmNTf32.apply(kn, kn) * dec * beta.unsqueeze(-1)).masked_fill(~strict, 0.0)
    Tm = unit_lower_inverse(A)
    u = (Tm * beta.unsqueeze(-2)).to(q.dtype) @ vc                       # (I + A)⁻¹ · diag(β) · v
    w = (Tm * (beta * torch.exp(gc)).unsqueeze(-2)).to(q.dtype) @ kn     # (I + A)⁻¹ · diag(β·exp(gc)) · k̂
    qk = (_BmmNTf32.apply(qn, kn) * dec).masked_fill(~incl, 0.0)
    o = _chunk_core(w, u, kd, qg, qk, torch.exp(gc[..., -1]))            # (B·H, nC, c, Dv)
    return o.reshape(B, H, Tp, Dv).permute(0, 2, 1, 3)[:, :T].to(v.dtype)


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
    scale = Dk ** -0.5 if scale is None else scale
    if _prepare_kernel_ok(q, k, v, chunk, l2norm):
        return _chunk_fused_prepare(q, k, v, g, beta, scale)
    pad = (-T) % chunk
    if pad:
        q, k, v = (F.pad(t, (0, 0, 0, 0, 0, pad)) for t in (q, k, v))
        g, beta = (F.pad(t, (0, 0, 0, pad)) for t in (g, beta))
    Tp = T + pad
    nC = Tp // chunk
    # (B·H,nC,c,·): the strided copy moves the input dtype (bf16 in training), the fp32 math starts after it
    r = lambda t: t.permute(0, 2, 1, 3).reshape(B * H, nC, chunk, t.shape[-1]).float()
    q, k, v = r(q), r(k), r(v)
    g, beta = g.float(), beta.float()
    if l2norm:
        q, k = _l2norm(q), _l2norm(k)
    q = q * scale
    g = g.permute(0, 2, 1).reshape(B * H, nC, chunk)
    beta = beta.permute(0, 2, 1).reshape(B * H, nC, chunk)
    gc = torch.cumsum(g, dim=-1)                                         # inclusive log-decay inside the chunk
    kb = k * beta.unsqueeze(-1)
    vb = v * beta.unsqueeze(-1)
    dec = torch.exp(gc.unsqueeze(-1) - gc.unsqueeze(-2))                 # [i,j] = exp(gc_i - gc_j)
    strict = torch.tril(torch.ones(chunk, chunk, device=q.device, dtype=torch.bool), -1)
    incl = torch.tril(torch.ones(chunk, chunk, device=q.device, dtype=torch.bool), 0)
    A = ((kb @ k.transpose(-1, -2)) * dec).masked_fill(~strict, 0.0)
    # (I + A) is unit lower-triangular → W, U from its inverse:  (I+A) U = β v ; (I+A) W = β k·exp(gc)
    Tm = unit_lower_inverse(A)
    u = Tm @ vb
    w = Tm @ (kb * torch.exp(gc).unsqueeze(-1))
    qk = ((q @ k.transpose(-1, -2)) * dec).masked_fill(~incl, 0.0)
    g_last = gc[..., -1]
    kd = k * torch.exp(g_last.unsqueeze(-1) - gc).unsqueeze(-1)          # keys decayed to the end of their chunk
    qg = q * torch.exp(gc).unsqueeze(-1)                                 # queries decayed from the chunk start
    o = _chunk_core(w, u, kd, qg, qk, torch.exp(g_last))                 # (B·H,nC,c,Dv)
    o = o.reshape(B, H, Tp, Dv).permute(0, 2, 1, 3)[:, :T]
    return o.to(dtype)


def gated_delta_rule(q, k, v, g, beta, scale: Optional[float] = None, l2norm: bool = True,
                     cu_seqlens: Optional[torch.Tensor] = None):
    return gated_delta_rule_chunk(q, k, v, g, beta, scale, l2norm, cu_seqlens)
