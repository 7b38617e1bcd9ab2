"""Mixture-of-experts building blocks: router, routing metadata, grouped expert FFN, aux loss.

Behavioural reference: `lit_gpt/smoe_functional.py:15-83` (token-choice router: top-k on the
logits, softmax over the selected k, optional ``sqrt(score + 1e-30)``; gather-fused grouped
up-projection + SwiGLU; grouped down-projection + score-weighted combine),
`lit_gpt/moe.py:33-39` (``stable_topk``: ties go to the lower expert index) and
`lit_gpt/aux_loss.py:151-171` (switch / entropy load-balance loss with optional global
all-reduce of both statistics).

GLU layout: **chunk halves** everywhere (``w_in[e]`` rows ``[0, I)`` are the gate, ``[I, 2I)``
the up projection), the same as the dense MLP and the shared expert of the reference
(`lit_gpt/moe.py:96-99`); upstream SonicMoE's interleaved layout is not used.

CUDA path: ``csrc/moe_routing.cu`` (top-k indices, slot layout, row gather / score-weighted
combine, all without a host sync) and the grouped mode of the two-CTA GEMM in
``csrc/gemm2_bf16.cu`` (per-expert row ranges read from device-side offsets); ``grouped_gemm.py``
strings them together as one autograd function.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn.functional as F

from . import backend
from .activations import swiglu_ref


# ------------------------------------------------------------------ router
def stable_topk(x: torch.Tensor, k: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """top-k along the last dim with ties broken towards the lower index."""
    order = torch.argsort(x, dim=-1, descending=True, stable=True)[..., :k]
    return torch.gather(x, -1, order), order


def router_topk_softmax_ref(logits: torch.Tensor, k: int, sqrt_gate: bool = False):
    vals, idx = stable_topk(logits.float(), k)
    scores = torch.softmax(vals, dim=-1)
    if sqrt_gate:
        scores = torch.sqrt(scores + 1e-30)
    return scores, idx.to(torch.int32)


def router_topk_softmax(logits: torch.Tensor, k: int, sqrt_gate: bool = False):
    """(N,E) logits → (scores (N,k) fp32 with grad, indices (N,k) int32).

    The selection (the expensive part) is one kernel; the softmax over the k selected logits is a
    gather + softmax on an (N,k) tensor, differentiable through plain autograd."""
    if (logits.is_cuda and logits.dtype == torch.float32 and logits.shape[1] <= 256 and backend.has("topk_indices")
            and backend.use_cuda_kernel("router", logits)):
        idx = backend.require_extension().topk_indices(logits.detach().contiguous(), k)
        backend.count_launch()
        vals = torch.gather(logits, 1, idx.long())
        scores = torch.softmax(vals, dim=-1)
        if sqrt_gate:
            scores = torch.sqrt(scores + 1e-30)
        return scores, idx
    return router_topk_softmax_ref(logits, k, sqrt_gate)


# ------------------------------------------------------------------ metadata
def routing_metadata_ref(indices: torch.Tensor, n_experts: int):
    """Stable sort of the N·K (token, slot) pairs by expert.

    Returns ``counts (E,) int32``, ``offsets (E+1,) int32``, ``sorted_pair (N·K,) int32`` — the flat
    pair id ``token·K + slot`` at each expert-sorted position.
    """
    flat = indices.reshape(-1).long()
    order = torch.argsort(flat, stable=True)
    counts = torch.bincount(flat, minlength=n_experts).to(torch.int32)
    offsets = torch.zeros(n_experts + 1, dtype=torch.int32, device=indices.device)
    offsets[1:] = torch.cumsum(counts, 0)
    return counts, offsets, order.to(torch.int32)


def routing_metadata(indices: torch.Tensor, n_experts: int):
    return routing_metadata_ref(indices, n_experts)


# ------------------------------------------------------------------ expert FFN
def moe_ffn_ref(x: torch.Tensor, w_in: torch.Tensor, w_out: torch.Tensor, scores: torch.Tensor,
                indices: torch.Tensor, b_in: Optional[torch.Tensor] = None,
                b_out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Dense-loop oracle.  x:(N,C) w_in:(E,2I,C) w_out:(E,C,I) scores,indices:(N,K) → (N,C)."""
    N, C = x.shape
    E = w_in.shape[0]
    out = torch.zeros(N, C, dtype=torch.float32, device=x.device)
    for e in range(E):
        tok, slot = torch.nonzero(indices == e, as_tuple=True)
        if tok.numel() == 0:
            continue
        h = F.linear(x[tok].to(w_in.dtype), w_in[e], None if b_in is None else b_in[e])
        g, u = h.chunk(2, dim=-1)
        y = F.linear(swiglu_ref(g, u), w_out[e], None if b_out is None else b_out[e])
        out.index_add_(0, tok, y.float() * scores[tok, slot].float().unsqueeze(-1))
    return out.to(x.dtype)


def moe_ffn_sorted_torch(x, w_in, w_out, scores, indices, b_in=None, b_out=None):
    """Same math through the sorted layout (the data flow the CUDA kernels use)."""
    N, C = x.shape
    E = w_in.shape[0]
    K = indices.shape[1]
    counts, offsets, sorted_pair = routing_metadata_ref(indices, E)
    tok = (sorted_pair // K).long()
    xs = x[tok]
    sizes = counts.tolist()
    outs = []
    start = 0
    for e, n in enumerate(sizes):
        if n == 0:
            continue
        h = F.linear(xs[start:start + n].to(w_in.dtype), w_in[e], None if b_in is None else b_in[e])
        g, u = h.chunk(2, dim=-1)
        outs.append(F.linear(swiglu_ref(g, u), w_out[e], None if b_out is None else b_out[e]))
        start += n
    ys = torch.cat(outs, dim=0) if outs else xs.new_zeros(0, C)
    sc = scores.reshape(-1)[sorted_pair.long()].unsqueeze(-1)
    out = torch.zeros(N, C, dtype=torch.float32, device=x.device)
    out.index_add_(0, tok, ys.float() * sc.float())
    return out.to(x.dtype)


def moe_ffn(x, w_in, w_out, scores, indices, b_in=None, b_out=None, shared=None, alpha: float = 1.0):
    """Routed expert FFN; with ``shared`` (the shared expert's output, (N, C)) and ``alpha`` the result is
    ``alpha * (routed + shared)`` — the mix of `lit_gpt/moe.py:636-641` folded into the combine pass."""
    from . import grouped_gemm
    if grouped_gemm.supported(x, w_in, w_out, b_in, b_out) and backend.use_cuda_kernel("grouped_gemm", x, w_in, w_out) \
            and (shared is None or shared.dtype == x.dtype):
        return grouped_gemm.moe_ffn_cuda(x, w_in, w_out, scores, indices, shared, alpha)
    out = moe_ffn_sorted_torch(x, w_in, w_out, scores, indices, b_in, b_out)
    if shared is not None:
        out = out + shared
    return out if alpha == 1.0 else out * alpha


def segment_cu_seqlens(sorted_sequence_ids: torch.Tensor, tokens_per_expert: torch.Tensor):
    """Packed-attention segments of expert-sorted tokens: a new segment starts where the expert or the sequence id changes, so
    that an attention expert never attends across sequences (or into another expert's rows).  Returns (cu_seqlens int32
    [n_seg + 1], segment lengths int32 [n_seg]).  Same contract as the helper the reference pins in
    `tests/test_build_segment_cu_seqlen.py:4-48`; here one run-length pass over the combined (expert, sequence) key."""
    n = sorted_sequence_ids.numel()
    dev = sorted_sequence_ids.device
    if n == 0:
        return torch.zeros(1, dtype=torch.int32, device=dev), torch.empty(0, dtype=torch.int32, device=dev)
    seq = sorted_sequence_ids.reshape(-1).long()
    counts = tokens_per_expert.reshape(-1).long()
    expert = torch.repeat_interleave(torch.arange(counts.numel(), device=dev), counts, output_size=n) if counts.numel() \
        else torch.zeros(n, dtype=torch.long, device=dev)
    key = expert * (int(seq.max()) + 1) + seq
    _, lengths = torch.unique_consecutive(key, return_counts=True)
    cu = F.pad(torch.cumsum(lengths, 0), (1, 0)).to(torch.int32)
    return cu, lengths.to(torch.int32)


# ------------------------------------------------------------------ aux loss
class _DiffAllReduceSum(torch.autograd.Function):
    """all-reduce(SUM) whose backward is another all-reduce(SUM) (torch.distributed.nn semantics)."""

    @staticmethod
    def forward(ctx, t, group):
        import torch.distributed as dist
        ctx.group = group
        t = t.clone()
        dist.all_reduce(t, group=group)
        return t

    @staticmethod
    def backward(ctx, g):
        import torch.distributed as dist
        g = g.clone()
        dist.all_reduce(g, group=ctx.group)
        return g, None


def load_balance_loss(expert_probs: torch.Tensor, tokens_per_expert: torch.Tensor, gamma: float = 1.0,
                      eps: float = 1e-30, style: str = "switch", global_stats: bool = False,
                      seq_len: Optional[int] = None, group=None) -> torch.Tensor:
    """expert_probs:(T,E) softmax over all experts; tokens_per_expert:(E,) or (B,E) for ``switch_seq``."""
    import torch.distributed as dist
    T, E = expert_probs.shape
    if style == "switch_seq":
        assert seq_len is not None
        Bn = T // seq_len
        p = expert_probs.view(Bn, seq_len, E).sum(dim=1) + eps
        p = p / p.sum(dim=-1, keepdim=True)
        f = tokens_per_expert.float() / (tokens_per_expert.sum(dim=-1, keepdim=True) + eps)
        return gamma * (E * (f * p).sum(dim=-1)).mean()
    p = expert_probs.sum(dim=0)
    if global_stats and dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        p = _DiffAllReduceSum.apply(p, group)
    p = p + eps
    if style == "entropy":
        loss = (p * torch.log(p)).sum()
    elif style == "switch":
        f = tokens_per_expert.to(p.dtype)
        loss = (tokens_per_expert.shape[0] * p / p.sum() * f / f.sum()).sum()
    else:
        raise ValueError(f"unknown aux style {style!r}")
    return gamma * loss


def compute_tokens_per_expert_seq(indices: torch.Tensor, n_experts: int, seq_len: int) -> torch.Tensor:
    """indices:(T,K) → (B,E) per-sequence token counts."""
    T, K = indices.shape
    Bn = T // seq_len
    flat = indices.view(Bn, seq_len * K).long()
    out = torch.zeros(Bn, n_experts, dtype=torch.float32, device=indices.device)
    out.scatter_add_(1, flat, torch.ones_like(flat, dtype=torch.float32))
    return out


def activation_budget_loss(router_out: torch.Tensor, tau: float = 0.25, mask: Optional[torch.Tensor] = None,
                           lambda_budget: float = 1.0, eps: float = 1e-6, loss: str = "mse",
                           mode: str = "per_layer") -> torch.Tensor:
    """Budget loss of the token-skipping layer configurator (`lit_gpt/aux_loss.py:7-84`): pushes the expected active
    fraction towards ``tau``.  router_out: (B, L, T) keep-probabilities; ``mask``: (B, T) valid tokens.
    ``per_layer`` compares every layer's mean over tokens with ``tau``, ``per_sequence`` the mean over layers and tokens;
    ``loss`` is ``"mse"`` or ``"bce"``."""
    p = router_out.clamp(eps, 1 - eps)
    if mask is None:
        frac = p.mean(dim=2)                                              # (B, L)
    else:
        m = mask.to(p.dtype).clamp(0.0, 1.0).unsqueeze(1)                 # (B, 1, T)
        frac = (p * m).sum(dim=2) / m.sum(dim=(1, 2)).clamp_min(eps).unsqueeze(1)
    if mode == "per_sequence":
        frac = frac.mean(dim=1)                                           # (B,)
    elif mode != "per_layer":
        raise ValueError(f"unknown mode {mode!r}")
    target = torch.full_like(frac, tau)
    if loss == "bce":
        val = torch.nn.functional.binary_cross_entropy(frac.clamp(eps, 1 - eps), target)
    elif loss == "mse":
        val = torch.nn.functional.mse_loss(frac, target)
    else:
        raise ValueError(f"unknown loss {loss!r}")
    return lambda_budget * val
