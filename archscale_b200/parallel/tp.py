"""Tensor parallelism with sequence parallelism for dense transformer blocks.

The reference has no working tensor parallelism (its "tensor_parallel" mesh axis is the FSDP shard axis,
`pretrain.py:384-387`; the Mamba-2 ``ColumnParallelLinear`` hooks run with ``process_group=None``,
`lit_gpt/mamba2.py:104-109,147-152`).  This module provides the Megatron layout the vocabulary of those hooks
refers to:

* attention ``q_proj / k_proj / v_proj`` and the MLP up-projection ``w1`` are column-parallel (output features —
  whole heads, and matching gate/up halves — split over the ``tp`` ranks);
* ``attn.proj`` and the MLP down-projection ``w3`` are row-parallel (input features split);
* between blocks the residual stream, the norms and the embedding / head work on a 1/tp slice of the sequence.
  Entering a block half, the slice is all-gathered along the sequence (backward: reduce-scatter); leaving it,
  the row-parallel partial sums are reduce-scattered along the sequence (backward: all-gather).

Parameters that are not split (norm gains, QK-norm gains, embedding, head, biases of row-parallel layers) see only
part of the tokens or heads on each rank, so their gradients are partial sums: :func:`sync_replicated_grads`
adds them over the ``tp`` group once per optimizer step.  Split parameters carry ``_tp_sharded = True``.

Muon under tensor parallelism orthogonalises each rank's slice of a split matrix on its own (block-wise
Newton–Schulz); AdamW-family updates are identical to the unsplit model.

The collectives here are ``torch.distributed`` calls (NCCL on GPUs, gloo in the CPU tests).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from archscale_b200 import ops
from archscale_b200.models.layers import Linear
from . import dist_utils as du
from .mesh import Mesh


# ------------------------------------------------------------------------------------------ sequence collectives
def _gather_seq(x: torch.Tensor, group) -> torch.Tensor:
    """(B, T/tp, C) on every rank → (B, T, C), slices in rank order along dim 1."""
    w = dist.get_world_size(group)
    B, Tl, C = x.shape
    buf = torch.empty(w, B, Tl, C, dtype=x.dtype, device=x.device)
    du.all_gather_into(buf.view(-1), x.contiguous().view(-1), group=group)
    return buf.permute(1, 0, 2, 3).reshape(B, w * Tl, C)


def _reduce_scatter_seq(x: torch.Tensor, group) -> torch.Tensor:
    """(B, T, C) partial sums on every rank → this rank's (B, T/tp, C) slice of the total."""
    w = dist.get_world_size(group)
    B, T, C = x.shape
    Tl = T // w
    inp = x.view(B, w, Tl, C).permute(1, 0, 2, 3).contiguous()
    out = torch.empty(B, Tl, C, dtype=x.dtype, device=x.device)
    du.reduce_scatter_sum(out.view(-1), inp.view(-1), group=group)
    return out


class _GatherSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return _gather_seq(x, group)

    @staticmethod
    def backward(ctx, g):
        return _reduce_scatter_seq(g.contiguous(), ctx.group), None


class _ReduceScatterSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return _reduce_scatter_seq(x.contiguous(), group)

    @staticmethod
    def backward(ctx, g):
        return _gather_seq(g, ctx.group), None


def gather_sequence(x: torch.Tensor, group) -> torch.Tensor:
    return _GatherSeq.apply(x, group)


def reduce_scatter_sequence(x: torch.Tensor, group) -> torch.Tensor:
    return _ReduceScatterSeq.apply(x, group)


# ------------------------------------------------------------------------------------------ sharded layers
class RowParallelLinear(Linear):
    """``Linear`` over a slice of the input features; the partial products are summed over the ``tp`` group and
    scattered along the sequence.  The bias (not split) is added after the reduction."""

    tp_group = None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        w = self.weight
        g = getattr(w, "_fsdp_group", None)
        if g is not None and getattr(g, "ag_pending", False):
            w._fsdp_engine.finish_pending_gather(g)
        if w.dtype != x.dtype:
            w = w.to(x.dtype)
        y = reduce_scatter_sequence(ops.linear(x, w, None), self.tp_group)
        if self.bias is not None:
            y = y + self.bias.to(y.dtype)
        return y


def _new_param(t: torch.Tensor, like: nn.Parameter, sharded: bool) -> nn.Parameter:
    p = nn.Parameter(t.detach().clone().contiguous(), requires_grad=like.requires_grad)
    if sharded:
        p._tp_sharded = True
    return p


def _split_rows(lin: Linear, tp: int, r: int, blocks: int = 1) -> None:
    """Keep this rank's output features; ``blocks`` > 1 splits each of that many equal row blocks (gate | up)."""
    out_f, in_f = lin.weight.shape
    per = out_f // blocks
    assert per % tp == 0, f"{out_f} output features in {blocks} block(s) do not divide over tp={tp}"
    sl = per // tp
    w = lin.weight.view(blocks, per, in_f)[:, r * sl:(r + 1) * sl].reshape(blocks * sl, in_f)
    lin.weight = _new_param(w, lin.weight, True)
    if lin.bias is not None:
        b = lin.bias.view(blocks, per)[:, r * sl:(r + 1) * sl].reshape(-1)
        lin.bias = _new_param(b, lin.bias, True)
    lin.out_features = blocks * sl


def _to_row_parallel(lin: Linear, tp: int, r: int, group) -> RowParallelLinear:
    out_f, in_f = lin.weight.shape
    assert in_f % tp == 0
    sl = in_f // tp
    new = RowParallelLinear.__new__(RowParallelLinear)
    nn.Module.__init__(new)
    new.in_features, new.out_features = sl, out_f
    new.weight = _new_param(lin.weight[:, r * sl:(r + 1) * sl], lin.weight, True)
    new.bias = None if lin.bias is None else _new_param(lin.bias, lin.bias, False)
    new.mxfp8 = False
    new.tp_group = group
    return new


def _wrap_gather_input(module: nn.Module, group) -> None:
    inner = module.forward

    def forward(x, *args, **kwargs):
        return inner(gather_sequence(x, group), *args, **kwargs)

    module.forward = forward


def apply_tensor_parallel(model: nn.Module, mesh: Mesh) -> None:
    """Split the attention and MLP weights of every block of ``model`` over ``mesh.tp_group`` in place and switch
    the model to sequence-sliced activations between blocks.  Call before the FSDP engine flattens parameters."""
    from archscale_b200.models.attention import CausalSelfAttention
    from archscale_b200.models.gpt import LLaMAMLP
    tp, r, group = mesh.tp, mesh.tp_rank, mesh.tp_group
    if tp <= 1:
        return
    cfg = model.config
    assert cfg.separate_qkv and not cfg.gated_attn and not cfg.attn_norm and not cfg.ffn_norm, \
        "tensor parallelism covers blocks with separate q/k/v projections and no post-attention / FFN norm"
    assert cfg.n_head % tp == 0 and cfg.n_query_groups % tp == 0, "heads and KV groups must divide over tp"
    for block in model.transformer.h:
        attn, mlp = getattr(block, "attn", None), getattr(block, "mlp", None)
        if not isinstance(attn, CausalSelfAttention) or not isinstance(mlp, LLaMAMLP) or attn.yoco_cross or attn.use_da:
            raise NotImplementedError("tensor parallelism supports dense transformer blocks (self-attention + MLP) only")
        for name in ("q_proj", "k_proj", "v_proj"):
            _split_rows(getattr(attn, name), tp, r)
        attn.n_head //= tp
        attn.n_query_groups //= tp
        if hasattr(attn, "softmax_offset"):
            H = attn.softmax_offset.shape[0] // tp
            attn.softmax_offset = _new_param(attn.softmax_offset[r * H:(r + 1) * H], attn.softmax_offset, True)
        attn.proj = _to_row_parallel(attn.proj, tp, r, group)
        _wrap_gather_input(attn, group)
        _split_rows(mlp.w1, tp, r, blocks=1 if mlp.relu2 else 2)
        mlp.w3 = _to_row_parallel(mlp.w3, tp, r, group)
        _wrap_gather_input(mlp, group)
    model.tp_size, model.tp_rank, model.tp_group = tp, r, group


def sequence_slice(t: torch.Tensor, tp: int, r: int, dim: int = 1) -> torch.Tensor:
    n = t.shape[dim]
    assert n % tp == 0, f"sequence length {n} does not divide over tp={tp}"
    return t.narrow(dim, r * (n // tp), n // tp)


@torch.no_grad()
def sync_replicated_grads(engine, mesh: Mesh) -> None:
    """Sum, over the ``tp`` group, the gradient shards of parameters that are not split (see the module docstring).
    Works on the flat fp32 gradient shards of the FSDP engine; call once per optimizer step, before clipping."""
    if mesh.tp <= 1:
        return
    for g in engine.groups():
        if g.grad is None:
            continue
        mask = _replicated_mask(g)
        if mask is None:
            continue
        if mask is True:
            du.all_reduce_sum(g.grad, group=mesh.tp_group)
        else:
            part = g.grad * mask
            du.all_reduce_sum(part, group=mesh.tp_group)
            g.grad.mul_(1 - mask).add_(part)


def _replicated_mask(g):
    """None: every parameter of the flat group is split; True: none is; else a 0/1 fp32 mask over this rank's shard."""
    if hasattr(g, "_tp_rep_mask"):
        return g._tp_rep_mask
    rep = [not getattr(s.param, "_tp_sharded", False) for s in g.specs]
    if not any(rep):
        out = None
    elif all(rep):
        out = True
    else:
        lo, hi = g.shard_range()
        m = torch.zeros(hi - lo, dtype=torch.float32, device=g.grad.device)
        for s, is_rep in zip(g.specs, rep):
            if is_rep:
                a, b = max(s.offset, lo), min(s.offset + s.numel, hi)
                if b > a:
                    m[a - lo:b - lo] = 1.0
        out = m
    g._tp_rep_mask = out
    return out


def replicated_sq_norm_split(engine):
    """(Σ g² over split parameters, Σ g² over unsplit parameters) of this rank's gradient shards — the global
    gradient norm adds the first over the ``tp`` group and counts the second once."""
    dev = engine.device
    sq_split = torch.zeros((), dtype=torch.float32, device=dev)
    sq_rep = torch.zeros((), dtype=torch.float32, device=dev)
    for g in engine.groups():
        if g.grad is None:
            continue
        mask = _replicated_mask(g)
        sq = g.grad.float().pow(2)
        if mask is None:
            sq_split += sq.sum()
        elif mask is True:
            sq_rep += sq.sum()
        else:
            sq_rep += (sq * mask).sum()
            sq_split += (sq * (1 - mask)).sum()
    return sq_split, sq_rep
