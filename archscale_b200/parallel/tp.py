"""Tensor parallelism with sequence parallelism for dense transformer blocks.

The reference has no working tensor parallelism (its "tensor_parallel" mesh axis is the FSDP shard axis,
`pretrain.py:384-387`; the Mamba-2 ``ColumnParallelLinear`` hooks run with ``process_group=None``,
`lit_gpt/mamba2.py:104-109,147-152`).  This module provides the Megatron layout the vocabulary of those hooks
refers to:

* attention ``q_proj / k_proj / v_proj`` and the MLP up-projection ``w1`` are column-parallel (output features —
  whole heads, and matching gate/up halves — split over the ``tp`` ranks);
* ``attn.proj`` and the MLP down-projection ``w3`` are row-parallel (input features split);
* between blocks the residual stream, the norms and the embedding / head work on a contiguous 1/tp chunk of the
  flattened (batch · sequence) tokens.  Entering a block half, the chunks are all-gathered (backward:
  reduce-scatter); leaving it, the row-parallel partial sums are reduce-scattered (backward: all-gather).

Parameters that are not split (norm gains, QK-norm gains, embedding, head, biases of row-parallel layers) see only
part of the tokens or heads on each rank, so their gradients are partial sums: :func:`sync_replicated_grads`
adds them over the ``tp`` group once per optimizer step.  Split parameters carry ``_tp_sharded = True``.

Muon under tensor parallelism orthogonalises each rank's slice of a split matrix on its own (block-wise
Newton–Schulz); AdamW-family updates are identical to the unsplit model.

The collectives here are ``torch.distributed`` calls (NCCL on GPUs, gloo in the CPU tests).
"""
from __future__ import annotations

import os
from typing import Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from archscale_b200 import ops
from archscale_b200.models.layers import Linear
from . import dist_utils as du
from .mesh import Mesh


# ------------------------------------------------------------------------------------------ token collectives
# Between blocks a rank holds a contiguous 1/tp chunk of the flattened (batch·sequence) token order, shaped
# (1, B·T/tp, C): whole batch rows when tp divides B, a stretch of the sequence when B = 1.  Gathered buffers
# are therefore rank-major and contiguous — no permutes around the collectives (or the peer-memory kernels).
def _gather_tokens(x: torch.Tensor, group) -> torch.Tensor:
    """(1, n, C) on every rank → (1, tp·n, C), chunks in rank order."""
    w = dist.get_world_size(group)
    _, n, C = x.shape
    out = torch.empty(1, w * n, C, dtype=x.dtype, device=x.device)
    du.all_gather_into(out.view(-1), x.contiguous().view(-1), group=group)
    return out


def _reduce_scatter_tokens(x: torch.Tensor, group) -> torch.Tensor:
    """(1, tp·n, C) partial sums on every rank → this rank's (1, n, C) chunk of the total."""
    w = dist.get_world_size(group)
    _, N, C = x.shape
    out = torch.empty(1, N // w, C, dtype=x.dtype, device=x.device)
    du.reduce_scatter_sum(out.view(-1), x.contiguous().view(-1), group=group)
    return out


class _GatherTokens(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return _gather_tokens(x, group)

    @staticmethod
    def backward(ctx, g):
        return _reduce_scatter_tokens(g, ctx.group), None


class _ReduceScatterTokens(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return _reduce_scatter_tokens(x, group)

    @staticmethod
    def backward(ctx, g):
        return _gather_tokens(g, ctx.group), None


def gather_tokens(x: torch.Tensor, group) -> torch.Tensor:
    return _GatherTokens.apply(x, group)


def reduce_scatter_tokens(x: torch.Tensor, group) -> torch.Tensor:
    return _ReduceScatterTokens.apply(x, group)


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
        fused = getattr(self, "_tp_fused", None)
        if fused is not None and fused.rs_enabled and fused.usable_rs(x, w):
            y = _LinearRSFn.apply(x.reshape(-1, x.shape[-1]), w, fused, self.weight).unsqueeze(0)
        else:
            y = ops.linear(x, w, None)
            y = reduce_scatter_tokens(y.reshape(1, -1, y.shape[-1]), self.tp_group)
        if self.bias is not None:
            y = y + self.bias.to(y.dtype)
        return y


def _new_param(t: torch.Tensor, like: nn.Parameter, sharded: bool, split=None) -> nn.Parameter:
    """``split = (dim, blocks)`` records how the slice was cut from the whole tensor (checkpoints undo it):
    along ``dim``; for dim 0, ``blocks`` equal row blocks (gate | up) were each cut into ``tp`` pieces."""
    p = nn.Parameter(t.detach().clone().contiguous(), requires_grad=like.requires_grad)
    if sharded:
        p._tp_sharded = True
        p._tp_split = split if split is not None else (0, 1)
    return p


def tp_whole_shape(local_shape, split, tp: int):
    shape = list(local_shape)
    shape[split[0]] *= tp
    return torch.Size(shape)


def tp_assemble(parts, split) -> torch.Tensor:
    """Inverse of the physical slicing: ``parts`` are the ``tp`` ranks' slices in rank order."""
    dim, blocks = split
    if dim != 0 or blocks == 1:
        return torch.cat(parts, dim=dim)
    sl = parts[0].shape[0] // blocks
    rest = parts[0].shape[1:]
    return torch.cat([t.reshape(blocks, sl, *rest) for t in parts], dim=1).reshape(blocks * sl * len(parts), *rest)


def tp_slice(whole: torch.Tensor, split, tp: int, r: int) -> torch.Tensor:
    """This rank's slice of a whole (unsplit) tensor, cut the way :func:`apply_tensor_parallel` cuts it."""
    dim, blocks = split
    if dim != 0 or blocks == 1:
        n = whole.shape[dim] // tp
        return whole.narrow(dim, r * n, n)
    per = whole.shape[0] // blocks
    sl = per // tp
    rest = whole.shape[1:]
    return whole.reshape(blocks, per, *rest)[:, r * sl:(r + 1) * sl].reshape(blocks * sl, *rest)


def _split_rows(lin: Linear, tp: int, r: int, blocks: int = 1) -> None:
    """Keep this rank's output features; ``blocks`` > 1 splits each of that many equal row blocks (gate | up)."""
    out_f, in_f = lin.weight.shape
    per = out_f // blocks
    assert per % tp == 0, f"{out_f} output features in {blocks} block(s) do not divide over tp={tp}"
    sl = per // tp
    w = lin.weight.view(blocks, per, in_f)[:, r * sl:(r + 1) * sl].reshape(blocks * sl, in_f)
    lin.weight = _new_param(w, lin.weight, True, (0, blocks))
    if lin.bias is not None:
        b = lin.bias.view(blocks, per)[:, r * sl:(r + 1) * sl].reshape(-1)
        lin.bias = _new_param(b, lin.bias, True, (0, blocks))
    lin.out_features = blocks * sl


def _to_row_parallel(lin: Linear, tp: int, r: int, group) -> RowParallelLinear:
    out_f, in_f = lin.weight.shape
    assert in_f % tp == 0
    sl = in_f // tp
    new = RowParallelLinear.__new__(RowParallelLinear)
    nn.Module.__init__(new)
    new.in_features, new.out_features = sl, out_f
    new.weight = _new_param(lin.weight[:, r * sl:(r + 1) * sl], lin.weight, True, (1, 1))
    new.bias = None if lin.bias is None else _new_param(lin.bias, lin.bias, False)
    new.mxfp8 = new.nvfp4 = False
    new.tp_group = group
    return new


def _wrap_gather_input(module: nn.Module, group, model: nn.Module, first: Linear) -> None:
    """Gather the token chunks in front of ``module``.  With the peer-memory context attached (``model._tp_fused``)
    the gather is fused into the GEMM of ``first`` — the first column-parallel layer that consumes the gathered
    activations — and that layer then returns the product computed by the fused launch."""
    inner = module.forward

    def forward(x, *args, **kwargs):
        B, T = model._tp_batch_shape                 # set by GPT.forward for the current micro-batch
        fused = getattr(model, "_tp_fused", None)
        if fused is not None and fused.usable(x, first):
            w = first.weight
            g = getattr(w, "_fsdp_group", None)
            if g is not None and getattr(g, "ag_pending", False):
                w._fsdp_engine.finish_pending_gather(g)
            x_full, y = _AGLinearFn.apply(x.view(-1, x.shape[-1]), w.to(x.dtype) if w.dtype != x.dtype else w, fused, w)
            x_full = x_full.view(B, T, x.shape[-1])
            first._tp_stash = (x_full, y.view(B, T, -1))
            try:
                return inner(x_full, *args, **kwargs)
            finally:
                first._tp_stash = None
        return inner(gather_tokens(x, group).view(B, T, x.shape[-1]), *args, **kwargs)

    module.forward = forward


class ColumnParallelLinear(Linear):
    """Column-parallel ``Linear``; when the wrapper in front of it already produced this layer's output inside the
    fused all-gather→GEMM launch, returns that product instead of multiplying again."""

    _tp_stash = None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        st = self._tp_stash
        if st is not None and x is st[0]:
            y = st[1]
            return y if self.bias is None else y + self.bias.to(y.dtype)
        return super().forward(x)


def apply_tensor_parallel(model: nn.Module, mesh: Mesh) -> None:
    """Split the attention and MLP weights of every block of ``model`` over ``mesh.tp_group`` in place and switch
    the model to token-sliced activations between blocks.  Call before the FSDP engine flattens parameters."""
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
        attn.q_proj.__class__ = ColumnParallelLinear
        mlp.w1.__class__ = ColumnParallelLinear
        attn.n_head //= tp
        attn.n_query_groups //= tp
        if hasattr(attn, "softmax_offset"):
            H = attn.softmax_offset.shape[0] // tp
            attn.softmax_offset = _new_param(attn.softmax_offset[r * H:(r + 1) * H], attn.softmax_offset, True, (0, 1))
        attn.proj = _to_row_parallel(attn.proj, tp, r, group)
        _wrap_gather_input(attn, group, model, attn.q_proj)
        _split_rows(mlp.w1, tp, r, blocks=1 if mlp.relu2 else 2)
        mlp.w3 = _to_row_parallel(mlp.w3, tp, r, group)
        _wrap_gather_input(mlp, group, model, mlp.w1)
    model.tp_size, model.tp_rank, model.tp_group = tp, r, group


def token_slice(t: torch.Tensor, tp: int, r: int) -> torch.Tensor:
    """(B, T, ...) → this rank's chunk of the flattened token order, shaped (1, B·T/tp, ...)."""
    flat = t.reshape(1, t.shape[0] * t.shape[1], *t.shape[2:])
    n = flat.shape[1]
    assert n % tp == 0, f"{n} tokens do not divide over tp={tp}"
    return flat.narrow(1, r * (n // tp), n // tp)


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


# ------------------------------------------------------------------------------------------ peer-memory fused layers
class FusedTPContext:
    """Symmetric-heap buffers and bookkeeping for the fused tensor-parallel layers (``csrc/gemm_bf16.cu``):

    * ``ag_linear``: this rank's token chunk is staged in the heap; one launch pulls every rank's chunk over
      NVLink into a local gathered buffer and multiplies row blocks as they arrive (all-gather → GEMM);
    * ``linear_rs``: one launch computes the full partial product into the heap, other ranks' row blocks first,
      publishes per-row-block counters, then sums this rank's rows from all peers (GEMM → reduce-scatter).

    Staging / partial-product buffers alternate between two copies: a buffer written in call n was last read by
    the peers in call n−2, and every rank must have launched call n−1 (which follows its call n−2 in stream order)
    before this rank's call n−1 could finish.
    """

    def __init__(self, mesh: Mesh, device: torch.device, max_tokens: int, max_features: int, n_copy: int = 16) -> None:
        from .symm import SymmetricHeap
        self.mesh, self.device, self.n_copy = mesh, device, n_copy
        self.tp = mesh.tp
        # The fused GEMM→reduce-scatter is exact but its own-slice epilogue still waits on per-lane peer loads (measured
        # 0.63 ms against 0.45 ms for GEMM + NCCL reduce-scatter at 2 GPUs, d16 shapes), so row-parallel layers use it
        # only on request; the fused all-gather→GEMM (0.67 ms against 0.72 ms) is always on.
        self.rs_enabled = os.environ.get("ARCHSCALE_B200_TP_FUSED_RS", "0") == "1"
        self.max_tokens, self.max_features = max_tokens, max_features
        chunk = (max_tokens // self.tp) * max_features * 2
        part = max_tokens * max_features * 2
        cnt = (max_tokens // 128 + 1) * 4
        self.heap = SymmetricHeap(mesh.tp_group, 2 * (chunk + part + cnt) + 8 * 1024, device)
        self.ext = self.heap.ext
        self.stage_off = [self.heap.alloc(chunk) for _ in range(2)]
        self.part_off = [self.heap.alloc(part) for _ in range(2)]
        self.cnt_off = [self.heap.alloc(cnt) for _ in range(2)]
        self.cnt = [self.heap.tensor(o, (max_tokens // 128 + 1,), torch.int32) for o in self.cnt_off]
        self.flags = [torch.zeros((max_tokens * max_features * 2 + 256 * 1024 - 1) // (256 * 1024) + 1, dtype=torch.int32,
                                  device=device) for _ in range(2)]
        self.ag_calls = 0
        self.rs_calls = 0
        self.expect = [0, 0]
        self.rs_rows = [None, None]
        torch.cuda.synchronize(device)
        self.heap.barrier(0)

    # -- eligibility -------------------------------------------------------------------------
    def usable(self, x_local: torch.Tensor, first: Linear) -> bool:
        n, K = x_local.shape[-2] * (x_local.shape[0] if x_local.dim() == 3 else 1), x_local.shape[-1]
        return (x_local.is_cuda and x_local.dtype == torch.bfloat16 and K % 64 == 0 and K <= self.max_features
                and n * self.tp <= self.max_tokens and first.weight.shape[0] % 8 == 0 and backend_has("ag_a_gemm"))

    def usable_rs(self, a: torch.Tensor, w: torch.Tensor) -> bool:
        M = a.numel() // a.shape[-1]
        return (a.is_cuda and a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and M % (128 * self.tp) == 0
                and M <= self.max_tokens and w.shape[0] <= self.max_features and w.shape[0] % 8 == 0
                and a.shape[-1] % 8 == 0 and backend_has("gemm_rs"))

    # -- launches ----------------------------------------------------------------------------
    def ag_linear(self, x_local: torch.Tensor, w: torch.Tensor):
        """x_local (n, K) bf16, w (N, K) bf16 → (x_full (tp·n, K), y (tp·n, N))."""
        i = self.ag_calls & 1
        self.ag_calls += 1
        n, K = x_local.shape
        self.heap.tensor(self.stage_off[i], (n, K), torch.bfloat16).copy_(x_local)
        e = self.heap.post(8 + i)
        self.heap.wait(8 + i, e)
        x_full, y = self.ext.ag_a_gemm(self.heap.bases, self.stage_off[i], n, w, self.flags[i], (self.ag_calls + 1) // 2,
                                       self.heap.rank, self.n_copy)
        ops.backend.count_launch(3)
        return x_full, y

    def linear_rs(self, a: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        """a (M, K/tp) bf16, w (N, K/tp) bf16 → this rank's (M/tp, N) rows of Σ_ranks a·wᵀ."""
        i = self.rs_calls & 1
        self.rs_calls += 1
        M, N = a.shape[0], w.shape[0]
        if self.rs_rows[i] not in (None, M):
            # a different row count leaves some counters behind: restart them (all ranks take this branch together)
            torch.cuda.synchronize(self.device)
            self.heap.barrier(1)
            self.cnt[i].zero_()
            self.expect[i] = 0
            torch.cuda.synchronize(self.device)
            self.heap.barrier(1)
        self.rs_rows[i] = M
        self.expect[i] += 4 * ((N + 255) // 256)
        out = self.ext.gemm_rs(a, w, self.heap.bases, self.part_off[i], self.cnt_off[i], self.expect[i], self.heap.rank)
        ops.backend.count_launch()
        return out


def backend_has(sym: str) -> bool:
    return ops.backend.has(sym)


class _AGLinearFn(torch.autograd.Function):
    """(x_full, y) = (all-gather(x_local), all-gather(x_local) · wᵀ) in one launch; backward: the gradients reaching
    x_full from its other consumers and from y are summed and reduce-scattered."""

    @staticmethod
    def forward(ctx, x_local, w, fused, w_param):
        x_full, y = fused.ag_linear(x_local.contiguous(), w)
        ctx.save_for_backward(x_full, w)
        ctx.fused, ctx.w_param = fused, w_param
        return x_full, y

    @staticmethod
    def backward(ctx, dx_full, dy):
        x_full, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1]).contiguous()
        dxf = ops.gemm.matmul_nn(dy2, w)
        if dx_full is not None:
            dxf = dxf + dx_full.reshape(dxf.shape)
        dx_local = _reduce_scatter_tokens(dxf.unsqueeze(0), ctx.fused.mesh.tp_group).squeeze(0)
        dw = None
        mg = getattr(ctx.w_param, "main_grad", None)
        if mg is not None:
            ops.gemm.matmul_tn_acc_(mg, dy2, x_full)
        else:
            dw = ops.gemm.matmul_tn(dy2, x_full)
        return dx_local, dw, None, None


class _LinearRSFn(torch.autograd.Function):
    """this rank's rows of Σ_ranks a·wᵀ in one launch; backward all-gathers the incoming gradient chunks."""

    @staticmethod
    def forward(ctx, a, w, fused, w_param):
        a = a.contiguous()
        ctx.save_for_backward(a, w)
        ctx.fused, ctx.w_param = fused, w_param
        return fused.linear_rs(a, w)

    @staticmethod
    def backward(ctx, d_local):
        a, w = ctx.saved_tensors
        d_full = _gather_tokens(d_local.contiguous().unsqueeze(0), ctx.fused.mesh.tp_group).squeeze(0)
        da = ops.gemm.matmul_nn(d_full, w)
        dw = None
        mg = getattr(ctx.w_param, "main_grad", None)
        if mg is not None:
            ops.gemm.matmul_tn_acc_(mg, d_full, a)
        else:
            dw = ops.gemm.matmul_tn(d_full, a)
        return da, dw, None, None


def enable_fused_layers(model: nn.Module, mesh: Mesh, device: torch.device, max_tokens: int) -> Optional[FusedTPContext]:
    """Attach the peer-memory context so that the column- / row-parallel layers of ``model`` run the fused launches."""
    if mesh.tp <= 1 or device.type != "cuda":
        return None
    cfg = model.config
    feat = max(cfg.n_embd, 1)
    ctx = FusedTPContext(mesh, device, max_tokens, feat)
    model._tp_fused = ctx
    for mod in model.modules():
        if isinstance(mod, RowParallelLinear):
            mod._tp_fused = ctx
    return ctx
