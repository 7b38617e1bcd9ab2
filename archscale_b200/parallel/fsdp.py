"""Fully-sharded data parallel engine (the FSDP2 role of the reference, re-designed).

What the reference gets from ``torch.distributed.fsdp.fully_shard`` per ``Block`` plus the root
module with ``MixedPrecisionPolicy(param_dtype=bf16, reduce_dtype=fp32)``
(`pretrain.py:536-563,806-807,924-928`) is provided here by one explicit engine:

* every *unit* (each ``Block``; the root unit holds embeddings, final norm and head) owns flat
  **fp32 master shards** (1/world of the unit, flat 1-D sharding so that the all-gather output
  *is* the parameter storage — no copy-out), a cached low-precision copy of its shard, and an
  fp32 gradient shard;
* forward / backward: all-gather (low precision) into a pooled buffer on a communication
  stream, prefetching the next unit while the current one computes; after the unit's backward
  the unit's gradients are packed in fp32, reduce-scattered (sum in fp32), scaled by 1/world and
  accumulated into the gradient shard on a second stream;
* numerically sensitive parameters (``A_log``, ``D``, ``dt_bias`` …) travel in fp32;
* expert-parallel parameters (``_ep_local``) are never gathered: each rank owns its experts;
* hybrid sharding: with ``dp > 1`` the gradient shard is all-reduced over the replica group.

Collectives are either ``torch.distributed`` (NCCL on GPUs, gloo on CPU test ranks) or the
peer-memory kernels of :mod:`archscale_b200.parallel.symm` when ``fused_comm`` is on.
Optimizers consume the flat shards through :meth:`FSDPEngine.groups` and :meth:`FlatGroup.local_slices`.
"""
from __future__ import annotations

import contextlib
from dataclasses import dataclass, field
from typing import Callable, Dict, Iterable, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn

from archscale_b200.utils.param_groups import is_matrix_param

from . import dist_utils as du
from .mesh import Mesh

_FP32_NAME_HINTS = ("A_log", ".D", "dt_bias", "dt_proj.bias", "lambda_q", "lambda_k", "softmax_offset")


def _keep_fp32(name: str) -> bool:
    return any(name.endswith(h) or (h in name and h.startswith("lambda")) for h in _FP32_NAME_HINTS)


@dataclass
class ParamSpec:
    name: str            # fully-qualified name in the model
    param: nn.Parameter
    shape: torch.Size
    numel: int
    offset: int          # element offset inside the group's flat (unsharded) buffer


class BufferPool:
    """Re-uses gathered-parameter / gradient buffers; cross-stream safety through events."""

    def __init__(self) -> None:
        self._free: Dict[Tuple[int, torch.dtype, str], List[Tuple[torch.Tensor, Optional[object]]]] = {}

    def get(self, numel: int, dtype: torch.dtype, device, stream=None) -> torch.Tensor:
        key = (numel, dtype, str(device))
        lst = self._free.get(key)
        if lst:
            buf, ev = lst.pop()
            if ev is not None:
                (stream or torch.cuda.current_stream()).wait_event(ev)
            return buf
        return torch.empty(numel, dtype=dtype, device=device)

    def put(self, buf: torch.Tensor) -> None:
        ev = None
        if buf.is_cuda:
            ev = torch.cuda.Event()
            ev.record()
        self._free.setdefault((buf.numel(), buf.dtype, str(buf.device)), []).append((buf, ev))


class FlatGroup:
    """Parameters of one unit that share a gather dtype, stored as one flat sharded vector."""

    def __init__(self, specs: List[ParamSpec], dtype: torch.dtype, world: int, rank: int, group, device,
                 sharded: bool = True, align: int = 64) -> None:
        self.specs, self.dtype, self.device = specs, dtype, device
        self.sharded = sharded and world > 1
        self.world = world if self.sharded else 1
        self.rank = rank if self.sharded else 0
        self.group = group if self.sharded else None
        total = sum(s.numel for s in specs)
        self.numel = total
        mult = self.world * align
        self.padded = ((total + mult - 1) // mult) * mult
        self.shard_numel = self.padded // self.world
        self.master: Optional[torch.Tensor] = None     # fp32 (shard_numel,)
        self.shard_lp: Optional[torch.Tensor] = None   # gather dtype copy of master (None if dtype is fp32)
        self.grad: Optional[torch.Tensor] = None       # fp32 (shard_numel,), accumulated over micro-steps
        self.full: Optional[torch.Tensor] = None       # gathered (padded,) in gather dtype
        self.full_grad: Optional[torch.Tensor] = None
        self.gather_event = None
        self.lp_stale = True

    # -- construction --------------------------------------------------------------
    @torch.no_grad()
    def shard_from_params(self) -> None:
        flat = torch.zeros(self.padded, dtype=torch.float32, device=self.device)
        for s in self.specs:
            flat[s.offset:s.offset + s.numel].copy_(s.param.detach().reshape(-1).to(torch.float32))
        lo = self.rank * self.shard_numel
        self.master = flat[lo:lo + self.shard_numel].clone()
        del flat
        self.lp_stale = True

    def shard_range(self) -> Tuple[int, int]:
        lo = self.rank * self.shard_numel
        return lo, lo + self.shard_numel

    def local_slices(self):
        """Yield (spec, lo, hi, shard_lo) for the part of each parameter stored on this rank:
        parameter elements [lo, hi) live at ``master[shard_lo : shard_lo + hi - lo]``."""
        a, b = self.shard_range()
        for s in self.specs:
            lo, hi = max(s.offset, a), min(s.offset + s.numel, b)
            if lo < hi:
                yield s, lo - s.offset, hi - s.offset, lo - a

    def refresh_lp(self) -> torch.Tensor:
        if self.dtype == torch.float32:
            return self.master
        if self.shard_lp is None:
            self.shard_lp = torch.empty_like(self.master, dtype=self.dtype)
        if self.lp_stale:
            self.shard_lp.copy_(self.master)
            self.lp_stale = False
        return self.shard_lp

    def set_param_views(self, full: Optional[torch.Tensor]) -> None:
        for s in self.specs:
            if full is None:
                s.param.data = torch.empty(0, dtype=self.dtype, device=self.device)
            else:
                s.param.data = full[s.offset:s.offset + s.numel].view(s.shape)

    # The gathered buffer is ONE persistent tensor per group whose storage is shrunk to zero bytes
    # when the unit is resharded and grown again before the next gather.  Parameter views and the
    # tensors autograd saved for backward keep pointing at this storage object, so they see the
    # re-gathered values in backward (a pooled buffer would be recycled for another unit in between).
    def alloc_full(self) -> torch.Tensor:
        if self.full is None:
            self.full = torch.empty(self.padded, dtype=self.dtype, device=self.device)
            self._full_nbytes = self.full.untyped_storage().nbytes()
            self.set_param_views(self.full)
        elif self.full.untyped_storage().nbytes() == 0:
            self.full.untyped_storage().resize_(self._full_nbytes)
        return self.full

    def free_full(self) -> None:
        if self.full is not None and self.world > 1:
            self.full.untyped_storage().resize_(0)


class Unit:
    def __init__(self, name: str, module: nn.Module, groups: List[FlatGroup], is_root: bool) -> None:
        self.name, self.module, self.groups, self.is_root = name, module, groups, is_root
        self.unsharded = False
        self.bwd_pending = False      # a backward for this unit is expected in the current step
        self.post_bwd_done = False


class _PostBackward(torch.autograd.Function):
    """Identity on the unit's inputs; its backward marks the end of the unit's backward pass."""

    @staticmethod
    def forward(ctx, engine, unit, *tensors):
        ctx.engine, ctx.unit = engine, unit
        return tensors if len(tensors) != 1 else tensors[0]

    @staticmethod
    def backward(ctx, *grads):
        ctx.engine._post_backward(ctx.unit)
        return (None, None) + grads


class FSDPEngine:
    def __init__(self, model: nn.Module, mesh: Optional[Mesh] = None, unit_classes: Sequence[type] = (),
                 param_dtype: torch.dtype = torch.bfloat16, reshard_after_forward: bool = True,
                 device: Optional[torch.device] = None, fused_comm: bool = False) -> None:
        self.model = model
        self.mesh = mesh or Mesh(world=1, rank=0, dp=1, fsdp=1, tp=1)
        self.world, self.rank, self.group = self.mesh.fsdp, self.mesh.fsdp_rank, self.mesh.fsdp_group
        self.param_dtype = param_dtype
        self.reshard_after_forward = reshard_after_forward and self.world > 1
        p0 = next(model.parameters())
        self.device = device or p0.device
        self.is_cuda = self.device.type == "cuda"
        self.pool = BufferPool()
        self.comm_stream = torch.cuda.Stream(self.device) if self.is_cuda else None
        self.rs_stream = torch.cuda.Stream(self.device) if self.is_cuda else None
        self.fused_comm = fused_comm and self.world > 1 and self.is_cuda
        self.fused_ag = self.fused_comm
        self.symm = None
        self.in_backward = False
        self.use_main_grad = self.is_cuda and param_dtype == torch.bfloat16
        self.requires_gradient_sync = True
        self.grad_scale = 1.0 / max(self.mesh.data_world, 1)
        self._rs_events: List[object] = []
        self._fwd_order: List[Unit] = []
        self._order_frozen = False
        self.units: List[Unit] = []
        self._build_units(unit_classes)
        self._register_hooks()
        if self.fused_comm:
            from . import symm
            self.symm = symm.SymmetricContext(self)
            for u in self.units:
                for g in u.groups:
                    first = g.specs[0] if g.specs else None
                    g.ag_pending = False
                    g.first_linear_ok = bool(first is not None and first.offset == 0 and len(first.shape) == 2
                                             and g.world > 1 and not u.is_root)
                    for sp in g.specs:
                        sp.param._fsdp_group = g
                        sp.param._fsdp_engine = self
                        sp.param._fsdp_first = sp is first

    # ------------------------------------------------------------------ construction
    def _build_units(self, unit_classes: Sequence[type]) -> None:
        model = self.model
        claimed: Dict[int, str] = {}
        unit_modules: List[Tuple[str, nn.Module]] = []
        for name, mod in model.named_modules():
            if unit_classes and isinstance(mod, tuple(unit_classes)):
                unit_modules.append((name, mod))
        named = dict(model.named_parameters(remove_duplicate=True))
        owner: Dict[int, Tuple[str, nn.Parameter]] = {}

        def make_unit(uname: str, mod: nn.Module, pnames: List[Tuple[str, nn.Parameter]], is_root: bool) -> Unit:
            buckets: Dict[Tuple[torch.dtype, bool], List[Tuple[str, nn.Parameter]]] = {}
            for n, p in pnames:
                local = bool(getattr(p, "_ep_local", False) or getattr(p, "_no_shard", False))
                dt = torch.float32 if (_keep_fp32(n) or self.param_dtype == torch.float32) else self.param_dtype
                # matrices (GEMM weights, Muon-managed) and vectors travel in separate flat groups: the matrix
                # group can then be gathered by the unit's first GEMM itself, after the norm weights are in place
                buckets.setdefault((dt, local, is_matrix_param(n, p.dim())), []).append((n, p))
            groups = []
            for (dt, local, _is_mat), items in sorted(buckets.items(), key=lambda kv: (not kv[0][2], str(kv[0][0]), kv[0][1])):
                specs, off = [], 0
                # matrices first: the Muon-managed part of every flat group is one contiguous prefix
                items = sorted(items, key=lambda it: 0 if is_matrix_param(it[0], it[1].dim()) else 1)
                for n, p in items:
                    specs.append(ParamSpec(n, p, p.shape, p.numel(), off))
                    off += p.numel()
                g = FlatGroup(specs, dt, self.world, self.rank, self.group, self.device, sharded=not local)
                g.ep_local = local
                g.matrix_numel = sum(s.numel for s in specs if is_matrix_param(s.name, len(s.shape)))
                g.shard_from_params()
                groups.append(g)
            return Unit(uname, mod, groups, is_root)

        for uname, mod in unit_modules:
            pn = []
            for n, p in mod.named_parameters(remove_duplicate=True):
                full = f"{uname}.{n}" if uname else n
                if id(p) in claimed:
                    continue
                claimed[id(p)] = full
                pn.append((full, p))
            if pn:
                self.units.append(make_unit(uname, mod, pn, False))
        rest = [(n, p) for n, p in named.items() if id(p) not in claimed]
        self.root = make_unit("", model, rest, True)
        self.units.append(self.root)
        # parameters now live in the shards; drop the full fp32 copies
        for u in self.units:
            for g in u.groups:
                g.set_param_views(None)
                if g.world > 1:
                    g.alloc_full()
                    g.free_full()

    def _register_hooks(self) -> None:
        for u in self.units:
            if u.is_root:
                u.module.register_forward_pre_hook(self._root_pre_forward, with_kwargs=True)
                u.module.register_forward_hook(self._root_post_forward)
            else:
                u.module.register_forward_pre_hook(lambda m, a, k, u=u: self._pre_forward(u, a, k), with_kwargs=True)
                u.module.register_forward_hook(lambda m, a, o, u=u: self._post_forward(u, o))

    # ------------------------------------------------------------------ gather / reshard
    def _unshard(self, unit: Unit, wait: bool = True) -> None:
        if not unit.unsharded:
            for g in unit.groups:
                lp = self.symm.lp_shard(g) if (self.symm is not None and g.world > 1) else g.refresh_lp()
                if g.world == 1:
                    if g.full is not lp:
                        g.full = lp
                        g.set_param_views(lp)
                    g.gather_event = None
                elif self.is_cuda and self._defer_to_first_gemm(unit, g, wait):
                    # fused path: the unit's first GEMM pulls the shards itself (ops.linear → symm.ag_gemm)
                    self.comm_stream.wait_stream(torch.cuda.current_stream())
                    with torch.cuda.stream(self.comm_stream):
                        g.alloc_full()
                        ev = torch.cuda.Event()
                        ev.record(self.comm_stream)
                    torch.cuda.current_stream().wait_event(ev)
                    g.ag_pending = True
                    g.gather_event = None
                elif self.is_cuda:
                    self.comm_stream.wait_stream(torch.cuda.current_stream())
                    with torch.cuda.stream(self.comm_stream):
                        g.alloc_full()
                        self._all_gather(g, lp)
                        g.gather_event = torch.cuda.Event()
                        g.gather_event.record(self.comm_stream)
                else:
                    g.alloc_full()
                    self._all_gather(g, lp)
            unit.unsharded = True
        if wait and self.is_cuda:
            for g in unit.groups:
                if g.gather_event is not None:
                    torch.cuda.current_stream().wait_event(g.gather_event)
                    g.gather_event = None

    def _defer_to_first_gemm(self, unit: Unit, g: FlatGroup, wait: bool) -> bool:
        """Forward of a non-root unit with peer-memory collectives: leave the matrix group to the fused
        all-gather→GEMM of the unit's first ``Linear``."""
        return (self.symm is not None and self.fused_ag and wait and not self.in_backward and not unit.is_root
                and g.dtype == torch.bfloat16 and getattr(g, "matrix_numel", 0) == g.numel and g.numel > 0
                and getattr(g, "first_linear_ok", False))

    def finish_pending_gather(self, g: FlatGroup) -> None:
        """Plain pull of a group whose gather was left to a GEMM that did not come first."""
        if getattr(g, "ag_pending", False):
            self._all_gather(g, g.shard_lp)
            g.ag_pending = False

    def _all_gather(self, g: FlatGroup, lp: torch.Tensor) -> None:
        if self.symm is not None:
            self.symm.all_gather(g, lp)
        else:
            du.all_gather_into(g.full, lp, group=g.group)

    def _reshard(self, unit: Unit) -> None:
        if not unit.unsharded:
            return
        for g in unit.groups:
            g.ag_pending = False
            if g.world > 1 and g.full is not None:
                if self.is_cuda:
                    # free on the communication stream, after the compute stream is done with the values
                    self.comm_stream.wait_stream(torch.cuda.current_stream())
                    with torch.cuda.stream(self.comm_stream):
                        g.free_full()
                else:
                    g.free_full()
        unit.unsharded = False

    # ------------------------------------------------------------------ hooks
    def _root_pre_forward(self, module, args, kwargs):
        if not self._order_frozen:
            self._fwd_order = []
        self._unshard(self.root)
        # first block gathers while embeddings run
        return None

    def _root_post_forward(self, module, args, output):
        self._order_frozen = True
        if not torch.is_grad_enabled():
            self._reshard_all()
        return None

    def _pre_forward(self, unit: Unit, args, kwargs):
        if not self._order_frozen and not self.in_backward:
            self._fwd_order.append(unit)
        self._unshard(unit)
        if not self.in_backward and not (self.symm is not None and self.fused_ag):
            # (with the fused all-gather→GEMM the next unit's first GEMM fetches its own parameters)
            nxt = self._neighbor(unit, +1)
            if nxt is not None:
                self._unshard(nxt, wait=False)
        if torch.is_grad_enabled() and not self.in_backward:
            unit.bwd_pending, unit.post_bwd_done = True, False
            tensors = [(i, a) for i, a in enumerate(args) if isinstance(a, torch.Tensor) and a.requires_grad]
            if tensors:
                outs = _PostBackward.apply(self, unit, *[a for _, a in tensors])
                outs = (outs,) if isinstance(outs, torch.Tensor) else outs
                args = list(args)
                for (i, _), o in zip(tensors, outs):
                    args[i] = o
                return tuple(args), kwargs
        return None

    def _post_forward(self, unit: Unit, output):
        if self.in_backward:
            return None  # recomputation inside backward: parameters are needed right away
        if torch.is_grad_enabled():
            def hook(grad, unit=unit):
                self._pre_backward(unit)
                return grad
            for t in _flatten_tensors(output):
                if t.requires_grad:
                    t.register_hook(hook)
        if self.reshard_after_forward:
            self._reshard(unit)
        return None

    def _neighbor(self, unit: Unit, step: int) -> Optional[Unit]:
        order = self._fwd_order
        if not self._order_frozen:
            return None
        try:
            i = order.index(unit)
        except ValueError:
            return None
        j = i + step
        return order[j] if 0 <= j < len(order) else None

    def _attach_main_grads(self, unit: Unit) -> None:
        """fp32 flat gradient buffers for the unit; ``Linear`` weight gradients are accumulated into
        them by the wgrad GEMM itself (``param.main_grad``), so no bf16 dW is ever materialised."""
        if not self.use_main_grad:
            return
        for g in unit.groups:
            self._ensure_full_grad(g)
            for s in g.specs:
                s.param.main_grad = g.full_grad[s.offset:s.offset + s.numel].view(s.shape)

    def _ensure_full_grad(self, g: FlatGroup) -> None:
        """Flat fp32 gradient buffer of the group for this micro-step (zeroed when it starts a new
        accumulation); with peer-memory collectives it is the group's buffer in the symmetric heap."""
        if g.full_grad is not None:
            return
        if self.symm is not None and g.world > 1:
            g.full_grad = g.symm_full_grad
            if not g.symm_fg_dirty:
                self.symm.wait_readers(g)        # peers may still pull the previous micro-step's slice (accumulation)
                g.full_grad.zero_()
                g.symm_fg_dirty = True
        else:
            g.full_grad = self.pool.get(g.padded, torch.float32, self.device)
            g.full_grad.zero_()

    def _pre_backward(self, unit: Unit) -> None:
        if unit.post_bwd_done:
            return
        self._unshard(unit)
        if not getattr(unit, "_mg_attached", False):
            self._attach_main_grads(unit)
            unit._mg_attached = True
        prv = self._neighbor(unit, -1)
        if prv is not None and prv.bwd_pending and not prv.post_bwd_done:
            self._unshard(prv, wait=False)

    def _post_backward(self, unit: Unit) -> None:
        if unit.post_bwd_done:
            return
        unit.post_bwd_done, unit.bwd_pending = True, False
        unit._mg_attached = False
        for g in unit.groups:
            for s in g.specs:
                if hasattr(s.param, "main_grad"):
                    del s.param.main_grad
        self._reduce_unit_grads(unit)
        if self.world > 1:
            self._reshard(unit)

    # ------------------------------------------------------------------ gradient reduction
    @torch.no_grad()
    def _reduce_unit_grads(self, unit: Unit) -> None:
        for g in unit.groups:
            have = [s for s in g.specs if s.param.grad is not None]
            if not have and g.full_grad is None:
                continue
            self._ensure_full_grad(g)
            if have:
                dst = [g.full_grad[s.offset:s.offset + s.numel].view(s.shape) for s in have]
                src = [s.param.grad for s in have]
                if all(t.dtype == torch.float32 for t in src):
                    torch._foreach_add_(dst, src)
                else:
                    torch._foreach_add_(dst, [t.to(torch.float32) for t in src])
                for s in have:
                    s.param.grad = None
            if not self.requires_gradient_sync:
                continue
            scale = self.grad_scale
            if g.world == 1:
                # not sharded: a single-process run, expert-parallel experts (each rank owns its
                # experts, gradients are already complete) or replicated parameters (all-reduce)
                fg, g.full_grad = g.full_grad, None
                if scale != 1.0:
                    fg.mul_(scale)
                if self.mesh.fsdp > 1 and not getattr(g, "ep_local", False):
                    du.all_reduce_sum(fg, group=self.mesh.fsdp_group)
                if self.mesh.dp > 1:
                    du.all_reduce_sum(fg, group=self.mesh.dp_group)
                if g.grad is None:
                    g.grad = fg
                else:
                    g.grad.add_(fg)
                    self.pool.put(fg)
                continue
            full_grad = g.full_grad
            g.full_grad = None
            if self.is_cuda:
                self.rs_stream.wait_stream(torch.cuda.current_stream())
                ctx = torch.cuda.stream(self.rs_stream)
            else:
                ctx = contextlib.nullcontext()
            with ctx:
                out = torch.empty(g.shard_numel, dtype=torch.float32, device=self.device)
                if self.symm is not None:
                    self.symm.reduce_scatter(g, out, full_grad, scale)
                else:
                    du.reduce_scatter_sum(out, full_grad, group=g.group)
                    out.mul_(scale)
                if self.mesh.dp > 1:
                    du.all_reduce_sum(out, group=self.mesh.dp_group)
                if g.grad is None:
                    g.grad = out
                else:
                    g.grad.add_(out)
                if self.is_cuda:
                    full_grad.record_stream(self.rs_stream)
                    ev = torch.cuda.Event()
                    ev.record(self.rs_stream)
                    self._rs_events.append(ev)
            if self.symm is not None:
                g.symm_fg_dirty = False      # consumed; the next micro-step starts from zero
            else:
                self.pool.put(full_grad)

    # ------------------------------------------------------------------ CPU offload of master / optimizer shards
    # The role of ``CPUOffloadPolicy`` in the reference (`pretrain.py:544`, ``--offloading`` / ``--fsdp_save_mem``), done
    # the other way round: the optimizer keeps running on the GPU, but between optimizer steps the fp32 master shards
    # and the optimizer's fp32 state shards (12 bytes per parameter and shard with Adam) live in pinned host memory, so
    # forward and backward — where activations peak — have that memory back.  Only the low-precision shard copy that the
    # all-gather reads stays on the device.  Groups that travel in fp32 (a few small vectors) are not offloaded.
    def enable_cpu_offload(self, state_dicts: Sequence[Dict[int, torch.Tensor]] = ()) -> None:
        """``state_dicts``: dicts ``id(group) → shard-shaped tensor`` owned by the optimizer (momentum, variance)."""
        self.cpu_offload = True
        self._off_dicts = list(state_dicts)
        self._off_host: Dict[Tuple[int, int], torch.Tensor] = {}
        self._offloaded = False

    def _to_host(self, key, t: torch.Tensor) -> torch.Tensor:
        h = self._off_host.get(key)
        if h is None or h.shape != t.shape or h.dtype != t.dtype:
            h = torch.empty(t.shape, dtype=t.dtype, device="cpu", pin_memory=self.is_cuda)
            self._off_host[key] = h
        h.copy_(t, non_blocking=True)
        return h

    @torch.no_grad()
    def offload_states(self) -> None:
        if not getattr(self, "cpu_offload", False) or self._offloaded:
            return
        for g in self.groups():
            if g.dtype == torch.float32 or g.master is None:
                continue
            if self.symm is not None and g.world > 1:
                self.symm.lp_shard(g)
            else:
                g.refresh_lp()                       # the forward pass gathers from this copy
            self._to_host((id(g), -1), g.master)
            g.master = None
            for k, d in enumerate(self._off_dicts):
                if id(g) in d and d[id(g)] is not None:
                    self._to_host((id(g), k), d[id(g)])
                    d[id(g)] = None
        if self.is_cuda:
            torch.cuda.current_stream().synchronize()   # host copies complete before the device tensors are released
        self._offloaded = True

    @torch.no_grad()
    def reload_states(self) -> None:
        if not getattr(self, "cpu_offload", False) or not self._offloaded:
            return
        for g in self.groups():
            h = self._off_host.get((id(g), -1))
            if h is None or g.master is not None:
                continue
            g.master = h.to(self.device, non_blocking=True)
            for k, d in enumerate(self._off_dicts):
                hk = self._off_host.get((id(g), k))
                if hk is not None and id(g) in d and d[id(g)] is None:
                    d[id(g)] = hk.to(self.device, non_blocking=True)
        self._offloaded = False

    # ------------------------------------------------------------------ public API
    def backward(self, loss: torch.Tensor) -> None:
        """``loss.backward()`` with unit-wise gather / reduce-scatter; returns after every
        gradient shard of this micro-step has been accumulated (on the compute stream)."""
        self.in_backward = True
        try:
            loss.backward()
        finally:
            self.in_backward = False
        for u in self.units:
            if u.is_root or (u.bwd_pending and not u.post_bwd_done):
                u.post_bwd_done, u.bwd_pending = True, False
                self._reduce_unit_grads(u)
        if self.world > 1:
            self._reshard_all()
        if self.is_cuda:
            for ev in self._rs_events:
                torch.cuda.current_stream().wait_event(ev)
            self._rs_events.clear()

    def _reshard_all(self) -> None:
        if self.world == 1:
            return
        for u in self.units:
            self._reshard(u)

    def unshard_all(self) -> None:
        for u in self.units:
            self._unshard(u)

    def set_requires_gradient_sync(self, flag: bool) -> None:
        self.requires_gradient_sync = flag

    def zero_grad(self) -> None:
        for u in self.units:
            for g in u.groups:
                g.grad = None

    def groups(self) -> Iterable[FlatGroup]:
        for u in self.units:
            yield from u.groups

    def mark_params_updated(self) -> None:
        """Call after the optimizer changed the master shards."""
        from archscale_b200.ops import mxfp8, nvfp4
        mxfp8.invalidate_weight_cache()          # quantised copies of the old weights are void
        nvfp4.invalidate_weight_cache()
        for g in self.groups():
            g.lp_stale = True
        for u in self.units:
            if u.unsharded and self.world == 1:
                for g in u.groups:
                    g.refresh_lp()
        if self.symm is not None:
            # publish the new shards in the symmetric heap, then meet the peers: after this barrier every
            # rank may pull any shard, and nobody still reads last step's gradient / Muon buffers
            for g in self.groups():
                if g.world > 1:
                    self.symm.lp_shard(g)
            self.symm.step_barrier()

    @torch.no_grad()
    def clip_grad_norm_(self, max_norm: float, eps: float = 1e-6, defer: bool = False):
        """Global L2 norm over all gradient shards (+ scale when above ``max_norm``);
        the role of ``fabric.clip_gradients`` (`pretrain.py:965-971`).  With ``defer=True`` the gradients are left
        untouched and ``(norm, coefficient)`` is returned: the optimizer multiplies the coefficient (a device scalar)
        into the gradients while it reads them (``ShardedOptimizer.step(grad_scale=...)``)."""
        # accumulators indexed [needs a sum over the fsdp group][parameter is split over the tp group]
        sq = [[torch.zeros((), dtype=torch.float32, device=self.device) for _ in range(2)] for _ in range(2)]
        grads = []
        tp_on = self.mesh.tp > 1
        if tp_on:
            from .tp import _replicated_mask
        for g in self.groups():
            if g.grad is None:
                continue
            grads.append(g.grad)
            fs = 1 if (g.world > 1 or getattr(g, "ep_local", False)) else 0
            mask = _replicated_mask(g) if tp_on else True
            if mask is True:
                sq[fs][0] += torch.linalg.vector_norm(g.grad, dtype=torch.float32).square()
            elif mask is None:
                sq[fs][1] += torch.linalg.vector_norm(g.grad, dtype=torch.float32).square()
            else:
                g2 = g.grad.float().pow(2)
                sq[fs][0] += (g2 * mask).sum()
                sq[fs][1] += (g2 * (1 - mask)).sum()
        if self.mesh.fsdp > 1:
            both = torch.stack(sq[1])
            du.all_reduce_sum(both, group=self.mesh.fsdp_group)
            sq[1] = [both[0], both[1]]
        rep, split = sq[0][0] + sq[1][0], sq[0][1] + sq[1][1]
        if tp_on:
            # tensor-parallel ranks hold different slices of the split matrices; unsplit parameters count once
            split = split.clone()
            du.all_reduce_sum(split, group=self.mesh.tp_group)
        total = torch.sqrt(rep + split)
        coef = None
        if max_norm is not None and max_norm > 0:
            coef = torch.clamp(max_norm / (total + eps), max=1.0)
            if grads and not defer:
                torch._foreach_mul_(grads, coef)
        return (total, coef) if defer else total

    # -- checkpoint support ----------------------------------------------------------
    # Checkpoints hold WHOLE tensors under the model's own key names, whatever the parallel layout that wrote them:
    # flat shards are gathered over the shard group, tensor-parallel slices are reassembled over the tp group (undoing
    # the gate | up block cut), expert-parallel slabs are concatenated over the ep group.  Loading cuts the whole tensor
    # the same way for this rank.  The optimizer's per-parameter state goes through the same two functions.
    def consolidate(self, spec: ParamSpec, g: FlatGroup, full_flat: torch.Tensor) -> torch.Tensor:
        """Whole tensor of ``spec`` from the group's gathered flat buffer (collective over tp / ep groups)."""
        t = full_flat[spec.offset:spec.offset + spec.numel].view(spec.shape)
        split = getattr(spec.param, "_tp_split", None)
        if split is not None and self.mesh.tp > 1:
            from .tp import tp_assemble
            parts = [torch.empty_like(t) for _ in range(self.mesh.tp)]
            torch.distributed.all_gather(parts, t.contiguous(), group=self.mesh.tp_group)
            t = tp_assemble(parts, split)
        if getattr(g, "ep_local", False) and self.mesh.ep > 1:
            # every rank owns different experts: concatenate the slabs along the expert dim
            parts = [torch.empty_like(t) for _ in range(self.mesh.ep)]
            torch.distributed.all_gather(parts, t.contiguous(), group=self.mesh.ep_group)
            t = torch.cat(parts, dim=0)
        return t

    def localize(self, spec: ParamSpec, g: FlatGroup, t: torch.Tensor) -> torch.Tensor:
        """This rank's (tp / ep-local) tensor of ``spec``, flattened, from a whole checkpoint tensor; raises when the
        checkpoint tensor has neither the whole nor the local number of elements."""
        split = getattr(spec.param, "_tp_split", None)
        tp_on = split is not None and self.mesh.tp > 1
        ep_on = getattr(g, "ep_local", False) and self.mesh.ep > 1
        whole = list(spec.shape)
        if tp_on:
            whole[split[0]] *= self.mesh.tp
        if ep_on:
            whole[0] *= self.mesh.ep
        n_whole = 1
        for d in whole:
            n_whole *= d
        if t.numel() == n_whole and (tp_on or ep_on):
            t = t.reshape(whole)
            if ep_on:
                n_local = whole[0] // self.mesh.ep
                t = t[self.mesh.ep_rank * n_local:(self.mesh.ep_rank + 1) * n_local]
            if tp_on:
                from .tp import tp_slice
                t = tp_slice(t, split, self.mesh.tp, self.mesh.tp_rank)
        elif t.numel() != spec.numel:
            raise ValueError(f"checkpoint tensor {spec.name} has {t.numel()} elements; expected {n_whole} (whole) "
                             f"or {spec.numel} (this rank's slice)")
        elif tp_on or ep_on:
            raise ValueError(f"checkpoint tensor {spec.name} holds one rank's slice ({t.numel()} elements), not the whole "
                             f"tensor ({n_whole}); it was written by a version that did not consolidate tp / ep slices")
        return t.reshape(-1)

    @torch.no_grad()
    def full_state_dict(self, rank0_only: bool = True, dtype: Optional[torch.dtype] = None) -> Dict[str, torch.Tensor]:
        """Consolidated fp32 (or ``dtype``) state dict with the model's own key names and whole-model shapes, on CPU."""
        out: Dict[str, torch.Tensor] = {}
        keep = (not rank0_only) or self.mesh.rank == 0
        self.reload_states()
        for g in self.groups():
            full = self._gather_master(g.master, g)
            for s in g.specs:
                t = self.consolidate(s, g, full)
                if keep:
                    out[s.name] = (t.to(dtype) if dtype else t).cpu().clone()
            del full
        # tied / duplicate names (e.g. lm_head.weight tied to wte.weight) and buffers
        if keep:
            seen = {id(p): n for n, p in self.model.named_parameters(remove_duplicate=True)}
            for n, p in self.model.named_parameters(remove_duplicate=False):
                if n not in out and id(p) in seen and seen[id(p)] in out:
                    out[n] = out[seen[id(p)]]
            for n, b in self.model.named_buffers():
                out[n] = b.detach().cpu().clone()
        return out

    def _gather_master(self, shard: torch.Tensor, g: FlatGroup) -> torch.Tensor:
        if g.world == 1:
            return shard
        full = torch.empty(g.padded, dtype=shard.dtype, device=self.device)
        du.all_gather_into(full, shard.contiguous(), group=g.group)
        return full

    @torch.no_grad()
    def load_full_state_dict(self, sd: Dict[str, torch.Tensor], strict: bool = True) -> None:
        missing = []
        self.reload_states()
        self.master_version = getattr(self, "master_version", 0) + 1      # cached norms of the old weights are void
        from archscale_b200.ops import mxfp8, nvfp4
        mxfp8.invalidate_weight_cache()
        nvfp4.invalidate_weight_cache()
        for g in self.groups():
            for s, lo, hi, slo in g.local_slices():
                if s.name not in sd:
                    missing.append(s.name)
                    continue
                src = self.localize(s, g, sd[s.name])[lo:hi]
                g.master[slo:slo + hi - lo].copy_(src.to(torch.float32))
            g.lp_stale = True
        if strict and missing:
            raise KeyError(f"missing keys in checkpoint: {missing[:8]}{'…' if len(missing) > 8 else ''}")
        self._reshard_all()
        for u in self.units:
            if u.unsharded:
                for g in u.groups:
                    g.refresh_lp()


def _flatten_tensors(obj) -> List[torch.Tensor]:
    if isinstance(obj, torch.Tensor):
        return [obj]
    if isinstance(obj, (list, tuple)):
        out: List[torch.Tensor] = []
        for o in obj:
            out.extend(_flatten_tensors(o))
        return out
    if isinstance(obj, dict):
        out = []
        for o in obj.values():
            out.extend(_flatten_tensors(o))
        return out
    return []
