"""Hybrid Muon / MuonH / AdamW / Adam-H optimizer working directly on the FSDP flat shards.

Role of `lit_gpt/optim/muon.py:27-650` + `scalar_opts.py:380-443` + `pretrain.py:565-592,
642-697` in the reference, re-designed around the flat shards of
:class:`archscale_b200.parallel.fsdp.FSDPEngine`:

* parameter classes follow the reference name rule: names without ``"weight"`` or containing
  any of ``conv1d wte lm_head norm ln layernorm`` are *vectors* (AdamW; 2-D ones get the
  Adam-hyperball step under MuonH except ``wte``), the rest are *matrices* (Muon);
* the whole model is processed as one batch per step (no per-parameter generator tasks):
  momentum update on the local shard slices → every matrix is assembled on one owner rank →
  Newton–Schulz on the owner (same-shape matrices batched) → orthogonalised updates return to
  the shards → MuonH norms are partial sums over local slices + **two** tiny all-reduces for the
  whole model (the reference issues three per parameter batch);
* expert tensors ``(E, out, in)`` are E independent matrices; each keeps its own norm under
  MuonH (the reference normalises the local slab as a whole, which makes the result depend on the expert-parallel degree);
* state (``momentum``, ``variance``) lives in fp32 buffers aligned with the master shards, so
  checkpoints consolidate it with the same gather as the weights.

Transport of matrices between shards and owners is pluggable: ``torch.distributed``
(all-gather + reduce-scatter; works on gloo) or the peer-memory kernels of
:mod:`archscale_b200.parallel.symm`.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from archscale_b200 import ops
from archscale_b200.optim import scalar_opts
from archscale_b200.parallel import dist_utils as du
from archscale_b200.parallel.fsdp import FlatGroup, FSDPEngine, ParamSpec

from archscale_b200.utils.param_groups import VECTOR_NAMES, is_vector_param  # noqa: E402,F401


@dataclass
class _Mat:
    """One 2-D matrix handled by Muon (a whole 2-D parameter or one expert of a 3-D tensor)."""
    group: FlatGroup
    spec: ParamSpec
    sub: int            # expert index inside a 3-D parameter (0 for 2-D)
    rows: int
    cols: int
    offset: int         # element offset inside the group's flat buffer
    owner: int          # rank (inside the shard group) that orthogonalises it
    norm_idx: int       # slot in the global norm vectors


class ShardedOptimizer:
    def __init__(self, engine: FSDPEngine, lr: float = 1e-3, betas: Tuple[float, float] = (0.9, 0.95),
                 eps: float = 1e-8, weight_decay: float = 0.0, vector_weight_decay: float = 0.0,
                 weight_lr_mult: float = 1.0, algorithm: str = "adamw", mu: float = 0.95, nesterov: bool = True,
                 adjust_lr: Optional[str] = "spectral_norm", ns_epsilon: float = 1e-8,
                 hyperball_exclude: Sequence[str] = ("transformer.wte.weight",), split_groups: bool = True,
                 vector_betas: Optional[Tuple[float, float]] = None, vector_eps: Optional[float] = None) -> None:
        """algorithm: "adamw" | "muon" | "muonh" | "lion" | "hadam".  ``split_groups=False`` applies AdamW with
        ``weight_decay`` to every parameter (the non-μP branch of the reference).  "hadam" is the reference's
        AdamW-for-vectors + NAdam-for-weights pair (`pretrain.py:646-654`): vectors use ``vector_betas`` /
        ``vector_eps`` (default ``betas`` / ``eps``), weight matrices the NAdam rule with ``betas`` / ``eps``."""
        assert algorithm in ("adamw", "muon", "muonh", "lion", "hadam")
        self.engine, self.lr, self.betas, self.eps = engine, lr, betas, eps
        self.vector_betas, self.vector_eps = vector_betas, vector_eps
        self.nadam_mu_product = 1.0
        self.weight_decay, self.vector_weight_decay = weight_decay, vector_weight_decay
        self.weight_lr_mult, self.algorithm = weight_lr_mult, algorithm
        self.mu, self.nesterov, self.adjust_lr, self.ns_epsilon = mu, nesterov, adjust_lr, ns_epsilon
        self.hyperball_exclude = set(hyperball_exclude)
        self.split_groups = split_groups
        self.step_count = 0
        self.use_muon = algorithm in ("muon", "muonh")
        self.use_muonh = algorithm == "muonh"
        # per-group state buffers aligned with the master shard
        self.m: Dict[int, torch.Tensor] = {}
        self.v: Dict[int, torch.Tensor] = {}
        self.mats: List[_Mat] = []
        self.hyper_vecs: List[Tuple[FlatGroup, ParamSpec, int]] = []   # Adam-H parameters (group, spec, norm_idx)
        self._classify()
        self.last_lrs: Dict[str, float] = {}
        self._norm_idx_cache: Dict[tuple, torch.Tensor] = {}
        # MuonH keeps every matrix on its sphere: after the renormalisation ‖X‖ is what it was before the step, so the
        # squared norms measured once stay valid until weights are loaded or weight decay shrinks them (one pass over
        # all master weights saved per step)
        self._xsq_cache: Optional[torch.Tensor] = None
        self._xsq_version = -1

    # ------------------------------------------------------------------ setup
    def _classify(self) -> None:
        n_norm = 0
        mats: List[_Mat] = []
        self.kind: Dict[int, str] = {}    # id(spec) -> "vector" (element-wise rule) | "matrix" (Muon)
        self.cls: Dict[int, str] = {}     # id(spec) -> "vector" | "matrix" by the name rule (lr mult / wd class)
        for g in self.engine.groups():
            gid = id(g)
            self.m[gid] = torch.zeros_like(g.master)
            need_v = False
            for s in g.specs:
                is_vec = is_vector_param(s.name) if self.split_groups else True
                self.cls[id(s)] = "vector" if is_vec else "matrix"
                elementwise = is_vec or len(s.shape) < 2 or not self.use_muon
                self.kind[id(s)] = "vector" if elementwise else "matrix"
                if elementwise:
                    need_v = True
                    if (self.use_muonh and len(s.shape) == 2 and is_vec and self.split_groups
                            and s.name not in self.hyperball_exclude):
                        self.hyper_vecs.append((g, s, n_norm))
                        n_norm += 1
                else:
                    rows, cols = s.shape[-2], s.shape[-1]
                    n_sub = s.numel // (rows * cols)
                    for e in range(n_sub):
                        mats.append(_Mat(g, s, e, rows, cols, s.offset + e * rows * cols, 0, n_norm))
                        n_norm += 1
            if need_v and self.algorithm != "lion":
                self.v[gid] = torch.zeros_like(g.master)
        # owners: biggest matrices first, round-robin → balanced Newton–Schulz work
        order = sorted(range(len(mats)), key=lambda i: -(mats[i].rows * mats[i].cols))
        load: Dict[Tuple[int, int], List[int]] = {}
        for i in order:
            mt = mats[i]
            w = mt.group.world
            key = (id(mt.group.group), w)
            if key not in load:
                load[key] = [0] * w
            r = min(range(w), key=lambda k: load[key][k])
            mt.owner = r
            load[key][r] += mt.rows * mt.cols * min(mt.rows, mt.cols)
        self.mats = mats
        self.n_norm = n_norm
        # norm slots of parameters that are complete on this rank (expert-parallel experts, replicated
        # tensors): they must not be summed over the shard group
        local = [mt.norm_idx for mt in mats if mt.group.world == 1] + [k for (g, _, k) in self.hyper_vecs if g.world == 1]
        self.local_norm_idx = torch.tensor(sorted(set(local)), dtype=torch.long, device=self.engine.device) if local else None

    # ------------------------------------------------------------------ helpers
    def _lr_for(self, kind: str) -> float:
        return self.lr * (self.weight_lr_mult if kind == "matrix" else 1.0)

    def _adjusted_lr(self, lr: float, rows: int, cols: int) -> float:
        if self.adjust_lr is None:
            return lr
        if self.adjust_lr == "spectral_norm":
            return lr * math.sqrt(rows / cols)
        if self.adjust_lr == "clip_norm":
            return lr * max(1.0, rows / cols) ** 0.5
        if self.adjust_lr == "rms_norm":
            return lr * 0.2 * math.sqrt(max(rows, cols))
        raise ValueError(self.adjust_lr)

    # ------------------------------------------------------------------ step
    @torch.no_grad()
    def step(self, lr: Optional[float] = None, weight_decay: Optional[float] = None,
             vector_weight_decay: Optional[float] = None, betas: Optional[Tuple[float, float]] = None,
             eps: Optional[float] = None, vector_betas: Optional[Tuple[float, float]] = None,
             vector_eps: Optional[float] = None, grad_scale: Optional[torch.Tensor] = None) -> None:
        """One update.  Every hyper-parameter passed here replaces the stored one from this step on (the trainer
        recomputes them per iteration: LR schedule, batch ramp-up, independent weight decay, beta schedules).
        ``grad_scale``: device scalar multiplied into every gradient on the fly (the gradient-clip coefficient of
        ``FSDPEngine.clip_grad_norm_(..., defer=True)``), so that clipping costs no pass over the gradients."""
        if lr is not None:
            self.lr = lr
        if weight_decay is not None:
            self.weight_decay = weight_decay
        if vector_weight_decay is not None:
            self.vector_weight_decay = vector_weight_decay
        if betas is not None:
            self.betas = betas
        if eps is not None:
            self.eps = eps
        if vector_betas is not None:
            self.vector_betas = vector_betas
        if vector_eps is not None:
            self.vector_eps = vector_eps
        self.step_count += 1
        eng = self.engine
        eng.reload_states()          # no-op unless master / state shards were offloaded to the host
        dev = eng.device
        fused_ok = eng.is_cuda and ops.backend.has("adamw_fused_")
        if grad_scale is not None and not (fused_ok and ops.backend.has("muon_momentum_")):
            # no kernel takes the scale on the fly here (CPU ranks): apply it to the gradient shards once
            torch._foreach_mul_([g.grad for g in eng.groups() if g.grad is not None], grad_scale)
            grad_scale = None
        self._grad_scale = grad_scale
        x_sq = torch.zeros(max(self.n_norm, 1), dtype=torch.float32, device=dev)
        u_sq = torch.zeros_like(x_sq)
        pending_hyper: List[Tuple[torch.Tensor, torch.Tensor, int, float]] = []   # (x_slice, u_slice, norm_idx, lr)

        # ---- vectors: AdamW / Lion / Adam-H on the local slices
        hyper_idx = {id(s): k for (_, s, k) in self.hyper_vecs}
        buckets: Dict[tuple, List[Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]]] = {}
        v_betas = self.vector_betas if self.vector_betas is not None else self.betas
        v_eps = self.vector_eps if self.vector_eps is not None else self.eps
        for g in eng.groups():
            if g.grad is None:
                continue
            gid = id(g)
            for s, lo, hi, slo in g.local_slices():
                if self.kind[id(s)] != "vector":
                    continue
                n = hi - lo
                x, gr, m = g.master[slo:slo + n], g.grad[slo:slo + n], self.m[gid][slo:slo + n]
                v = self.v[gid][slo:slo + n] if gid in self.v else None
                is_vec_cls = self.cls[id(s)] == "vector" and self.split_groups
                lr_p = self.lr if is_vec_cls or not self.split_groups else self.lr * self.weight_lr_mult
                wd = self.vector_weight_decay if is_vec_cls else self.weight_decay
                bt, ep_ = (v_betas, v_eps) if is_vec_cls else (self.betas, self.eps)
                rule = "nadam" if (self.algorithm == "hadam" and not is_vec_cls) else self.algorithm
                # one-pass kernel for slices big enough to matter (embedding, head, …); small ones stay on foreach
                big = (fused_ok and v is not None and n >= (1 << 16) and n % 4 == 0 and slo % 4 == 0 and rule not in ("lion", "nadam")
                       and x.dtype == torch.float32 and gr.dtype == torch.float32)
                if id(s) in hyper_idx:
                    k = hyper_idx[id(s)]
                    if big and not wd:
                        u = torch.empty_like(x)
                        acc2 = torch.zeros(2, dtype=torch.float32, device=dev)
                        ops.backend.require_extension().adamw_fused_(1, x, gr, m, v, u, lr_p, bt[0], bt[1], ep_, 0.0, self.step_count,
                                                                     grad_scale, acc2)
                        ops.backend.count_launch()
                        x_sq[k] += acc2[0]
                        u_sq[k] += acc2[1]
                    else:
                        if grad_scale is not None:
                            gr = gr * grad_scale
                        u = scalar_opts.adamw_direction_([m], [v], [gr], bt[0], bt[1], ep_, self.step_count)[0]
                        if wd:
                            x.mul_(1 - lr_p * wd)
                        x_sq[k] += x.float().pow(2).sum()
                        u_sq[k] += u.float().pow(2).sum()
                    pending_hyper.append((x, u, k, lr_p))
                elif big:
                    ops.backend.require_extension().adamw_fused_(0, x, gr, m, v, None, lr_p, bt[0], bt[1], ep_, wd, self.step_count,
                                                                 grad_scale, None)
                    ops.backend.count_launch()
                else:
                    if grad_scale is not None:
                        gr = gr * grad_scale
                    buckets.setdefault((lr_p, wd, bt, ep_, rule), []).append((x, gr, m, v))
        for (lr_p, wd, bt, ep_, rule), items in buckets.items():
            xs, gs, ms, vs = (list(t) for t in zip(*items))
            if rule == "lion":
                scalar_opts.lion_update_foreach(xs, gs, ms, lr_p, bt[0], bt[1], wd)
            elif rule == "nadam":
                scalar_opts.nadam_update_foreach(xs, gs, ms, vs, lr_p, bt[0], bt[1], wd, self.step_count, ep_,
                                                 self.nadam_mu_product)
            else:
                scalar_opts.adamw_update_foreach(xs, gs, ms, vs, lr_p, bt[0], bt[1], wd, self.step_count, ep_)
        if self.algorithm == "hadam":
            # advance the product once per step on every rank (also on ranks whose shard holds no weight slice)
            self.nadam_mu_product *= scalar_opts.nadam_mu(self.betas[0], self.step_count)

        # ---- matrices: momentum on local slices, orthogonalise on owners, scatter back
        hb_x: List[torch.Tensor] = [t[0] for t in pending_hyper]
        hb_u: List[torch.Tensor] = [t[1] for t in pending_hyper]
        hb_k: List[int] = [t[2] for t in pending_hyper]
        hb_lr: List[float] = [t[3] for t in pending_hyper]
        seg_groups: List[Tuple[torch.Tensor, torch.Tensor, dict]] = []   # (master prefix, O prefix, tables): fused path
        lr_m = self._lr_for("matrix")
        xsq_cached = (self.use_muonh and not self.weight_decay and self._xsq_cache is not None
                      and self._xsq_version == getattr(eng, "master_version", 0))
        if self.mats:
            o_shards = self._orthogonalised_updates(u_sq)
            wd = self.weight_decay
            xs, os_, ks, adj = [], [], [], []
            fused_gids = set()
            for gid, g in {id(mt.group): mt.group for mt in self.mats}.items():
                tb = self._seg_tables(g) if g.grad is not None else None
                if tb is not None and o_shards[gid].dtype == torch.bfloat16:
                    n = tb["n"]
                    seg_groups.append((g.master[:n], o_shards[gid][:n], tb))
                    fused_gids.add(gid)
            for mt in self.mats:
                g = mt.group
                if g.grad is None or id(g) in fused_gids:
                    continue
                a, b = g.shard_range()
                lo, hi = max(mt.offset, a), min(mt.offset + mt.rows * mt.cols, b)
                if lo >= hi:
                    continue
                xs.append(g.master[lo - a:hi - a])
                os_.append(o_shards[id(g)][lo - a:hi - a])
                ks.append(mt.norm_idx)
                adj.append(-self._adjusted_lr(lr_m, mt.rows, mt.cols))
            if wd:
                for x, _, _ in seg_groups:
                    x.mul_(1 - lr_m * wd)
            if xs:
                if wd:
                    torch._foreach_mul_(xs, 1 - lr_m * wd)
                if self.use_muonh:
                    if not xsq_cached:
                        sq = torch.stack(torch._foreach_norm(xs)).square()
                        x_sq.index_add_(0, torch.tensor(ks, device=dev), sq)
                    hb_x += xs
                    hb_u += os_
                    hb_k += ks
                    hb_lr += [lr_m] * len(xs)
                else:
                    upd = torch._foreach_mul([o.to(x.dtype) for o, x in zip(os_, xs)], adj)
                    torch._foreach_add_(xs, upd)
            if seg_groups:
                ext = ops.backend.require_extension()
                if self.use_muonh:
                    if not xsq_cached:
                        for x, _, tb in seg_groups:
                            ext.seg_update_(0, x, None, tb["bounds"], tb["kidx"], None, x_sq)
                else:
                    for x, o, tb in seg_groups:          # plain Muon: x ← x − lr·sqrt(rows/cols)·O
                        ext.seg_update_(1, x, o, tb["bounds"], tb["kidx"], self._adjusted_lr_vector(lr_m), self._scratch_acc())
                    seg_groups = []
                ops.backend.count_launch(len(seg_groups))

        # ---- hyperball: global norms (2 all-reduces for the whole model), update, renormalise
        if hb_x or seg_groups:
            if eng.mesh.fsdp > 1:
                packed = torch.stack((x_sq, u_sq))
                keep = packed[:, self.local_norm_idx].clone() if self.local_norm_idx is not None else None
                du.all_reduce_sum(packed, group=eng.mesh.fsdp_group)
                if keep is not None:
                    packed[:, self.local_norm_idx] = keep
                x_sq, u_sq = packed[0], packed[1]
            if self.use_muonh and not self.weight_decay and self.mats:
                mat_idx = self._mat_norm_idx(dev)
                if xsq_cached:
                    x_sq[mat_idx] = self._xsq_cache[mat_idx]
                else:
                    self._xsq_cache, self._xsq_version = x_sq.clone(), getattr(eng, "master_version", 0)
            x_norm, u_norm = x_sq.sqrt(), u_sq.sqrt().clamp_min(self.ns_epsilon)
            ratio = x_norm / u_norm
            new_sq = torch.zeros_like(x_sq)
            if hb_x:
                kidx = torch.tensor(hb_k, device=dev)
                coef = ratio[kidx] * torch.tensor(hb_lr, device=dev, dtype=torch.float32)
                upd = [u.to(x.dtype) if u.dtype != x.dtype else u for u, x in zip(hb_u, hb_x)]
                upd = torch._foreach_mul(upd, list(coef.unbind(0)))
                torch._foreach_sub_(hb_x, upd)
                new_sq.index_add_(0, kidx, torch.stack(torch._foreach_norm(hb_x)).square())
            if seg_groups:
                ext = ops.backend.require_extension()
                coef_m = (ratio * lr_m).contiguous()
                for x, o, tb in seg_groups:
                    ext.seg_update_(1, x, o, tb["bounds"], tb["kidx"], coef_m, new_sq)
                ops.backend.count_launch(len(seg_groups))
            if eng.mesh.fsdp > 1:
                keep = new_sq[self.local_norm_idx].clone() if self.local_norm_idx is not None else None
                du.all_reduce_sum(new_sq, group=eng.mesh.fsdp_group)
                if keep is not None:
                    new_sq[self.local_norm_idx] = keep
            scale_v = (x_norm / new_sq.sqrt().clamp_min(self.ns_epsilon)).contiguous()
            if hb_x:
                torch._foreach_mul_(hb_x, list(scale_v[kidx].unbind(0)))
            if seg_groups:
                for x, _, tb in seg_groups:
                    ext.seg_update_(2, x, None, tb["bounds"], tb["kidx"], scale_v, None)
                ops.backend.count_launch(len(seg_groups))
        eng.mark_params_updated()

    # ------------------------------------------------------------------ fused segment kernels (CUDA)
    def _seg_tables(self, g):
        """Segment tables of group ``g`` for ``csrc/optim.cu``: the Muon matrices must tile the local prefix of the
        flat fp32 shard without gaps (they are the contiguous prefix of a block's flat group).  None → foreach path."""
        cache = self.__dict__.setdefault("_seg_cache", {})
        if id(g) in cache:
            return cache[id(g)]
        tb = None
        eng = self.engine
        if eng.is_cuda and g.master.dtype == torch.float32 and ops.backend.has("seg_update_"):
            a, b = g.shard_range()
            segs = []
            for mt in self.mats:
                if mt.group is not g:
                    continue
                lo, hi = max(mt.offset, a), min(mt.offset + mt.rows * mt.cols, b)
                if lo < hi:
                    segs.append((lo - a, hi - a, mt.norm_idx))
            segs.sort()
            ok = bool(segs) and segs[0][0] == 0 and all(segs[i][1] == segs[i + 1][0] for i in range(len(segs) - 1)) \
                and all(s[0] % 4 == 0 for s in segs) and segs[-1][1] % 4 == 0
            if ok:
                dev = eng.device
                tb = {"n": segs[-1][1],
                      "bounds": torch.tensor([s[0] for s in segs] + [segs[-1][1]], dtype=torch.int64, device=dev),
                      "kidx": torch.tensor([s[2] for s in segs], dtype=torch.int32, device=dev)}
        cache[id(g)] = tb
        return tb

    def _mat_norm_idx(self, dev) -> torch.Tensor:
        if getattr(self, "_mat_idx_t", None) is None:
            self._mat_idx_t = torch.tensor(sorted({mt.norm_idx for mt in self.mats}), dtype=torch.long, device=dev)
        return self._mat_idx_t

    def _adjusted_lr_vector(self, lr_m: float) -> torch.Tensor:
        """Per-matrix step sizes (slot = norm index) for the plain-Muon fused update."""
        v = torch.zeros(max(self.n_norm, 1), dtype=torch.float32)
        for mt in self.mats:
            v[mt.norm_idx] = self._adjusted_lr(lr_m, mt.rows, mt.cols)
        return v.to(self.engine.device)

    def _scratch_acc(self) -> torch.Tensor:
        return torch.zeros(max(self.n_norm, 1), dtype=torch.float32, device=self.engine.device)

    # ------------------------------------------------------------------ Muon transport + NS
    def _transport_tables(self, g):
        """(gather table, return table) of the peer-memory Muon transport for flat group ``g``, built once: which 16-byte
        ranges this rank pulls from which shard to assemble the matrices it owns, and from which owner it pulls each
        range of its own shard afterwards.  None if a range is not 16-byte aligned (the full gather is used then)."""
        cache = self.__dict__.setdefault("_transport_cache", {})
        if id(g) in cache:
            return cache[id(g)]
        S, r, W = g.shard_numel, g.rank, g.world
        mats = [mt for mt in self.mats if mt.group is g]
        gather, ret = [], []
        a0, b0 = r * S, min((r + 1) * S, g.matrix_numel)
        for mt in mats:
            lo, hi = mt.offset, mt.offset + mt.rows * mt.cols
            if mt.owner == r:
                for sh in range(lo // S, (hi - 1) // S + 1):
                    a, b = max(lo, sh * S), min(hi, (sh + 1) * S)
                    gather.append((sh, a - sh * S, a, b - a))
            a, b = max(lo, a0), min(hi, b0)
            if b > a:
                ret.append((mt.owner, a, a - a0, b - a))
        sym = self.engine.symm
        tg = sym._piece_table(gather, r, W, self.engine.device)
        tr = sym._piece_table(ret, r, W, self.engine.device)
        cache[id(g)] = None if (tg is None or tr is None) else (tg, tr)
        return cache[id(g)]

    def _orthogonalise(self, stack: torch.Tensor) -> torch.Tensor:
        """(B, rows, cols) pre-orthogonalisation updates → orthogonalised updates (overridden by MuonBall)."""
        return ops.newton_schulz(stack, epsilon=self.ns_epsilon)

    @torch.no_grad()
    def _orthogonalised_updates(self, u_sq: torch.Tensor) -> Dict[int, torch.Tensor]:
        """Returns {id(group): bf16/fp32 shard-shaped tensor with the orthogonalised update O};
        fills ``u_sq[norm_idx] = ‖O‖²`` (complete on every rank after the hyperball all-reduce)."""
        eng = self.engine
        groups = {id(mt.group): mt.group for mt in self.mats}
        cdt = torch.bfloat16 if eng.is_cuda else torch.float32
        out: Dict[int, torch.Tensor] = {}
        staged: Dict[int, tuple] = {}
        for gid, g in groups.items():
            if g.grad is None:
                continue
            # 1. momentum (fp32) and the pre-orthogonalisation update U on the local shard.  Matrices
            #    are the contiguous prefix [0, matrix_numel) of the flat group, so this is one slice.
            m = self.m[gid]
            mask_mats = [mt for mt in self.mats if mt.group is g]
            a, b = g.shard_range()
            # only the matrix ranges of U are ever read (by the owners' Newton–Schulz batches): the tail needs no fill
            if eng.symm is not None and g.world > 1:
                u_shard = eng.symm.u_buffer(g)
            else:
                u_shard = torch.empty(g.shard_numel, dtype=cdt, device=eng.device)
            n_loc = min(b, g.matrix_numel) - a
            if n_loc > 0:
                ms, gs = m[:n_loc], g.grad[:n_loc]
                if (eng.is_cuda and u_shard.dtype == torch.bfloat16 and ms.dtype == torch.float32 and gs.dtype == torch.float32
                        and n_loc % 4 == 0 and ops.backend.has("muon_momentum_")):
                    # one pass: momentum update, Nesterov combination and the bf16 cast of U
                    ops.backend.require_extension().muon_momentum_(gs, ms, u_shard[:n_loc], self.mu, self.nesterov,
                                                                   getattr(self, "_grad_scale", None))
                    ops.backend.count_launch()
                else:
                    if getattr(self, "_grad_scale", None) is not None:
                        gs = gs * self._grad_scale
                    ms.mul_(self.mu).add_(gs)
                    if self.nesterov:
                        u_shard[:n_loc].copy_(torch.add(gs, ms, alpha=self.mu))
                    else:
                        u_shard[:n_loc].copy_(ms)
            # 2. assemble whole matrices.  Peer-memory path: a rank pulls only the matrices it owns; collective path:
            #    every rank gets the full flat U and owners use their matrices.
            tabs = self._transport_tables(g) if (g.world > 1 and eng.symm is not None) else None
            if g.world > 1:
                if tabs is not None:
                    u_full = eng.symm.gather_owned(g, u_shard, tabs[0])
                elif eng.symm is not None:
                    u_full = eng.symm.gather_flat(g, u_shard)
                else:
                    u_full = torch.empty(g.padded, dtype=cdt, device=eng.device)
                    du.all_gather_into(u_full, u_shard, group=g.group)
            else:
                u_full = u_shard
            if g.world > 1 and eng.symm is not None:
                o_full = eng.symm.o_buffer(g)
                if tabs is None:
                    o_full.zero_()              # the summing return path reads every rank's whole buffer
            else:
                o_full = torch.zeros(g.padded, dtype=cdt, device=eng.device) if g.world > 1 else u_full
            staged[gid] = (g, u_full, o_full, [mt for mt in mask_mats if mt.owner == g.rank])
        # 3. Newton–Schulz on owned matrices: one batch per shape over ALL groups (the same projection of every layer),
        #    so that the batched GEMMs fill whole waves of CTAs and the launch count does not grow with depth.  Runs of
        #    matrices stored back to back (the experts of one 3-D parameter, sibling projections) enter as one view.
        by_shape: Dict[Tuple[int, int], List[Tuple[int, List[_Mat]]]] = {}
        for gid, (g, u_full, o_full, mine) in staged.items():
            per: Dict[Tuple[int, int], List[_Mat]] = {}
            for mt in mine:
                per.setdefault((mt.rows, mt.cols), []).append(mt)
            for shape, lst in per.items():
                lst = sorted(lst, key=lambda mt: mt.offset)
                run = [lst[0]]
                for mt in lst[1:]:
                    if mt.offset == run[-1].offset + shape[0] * shape[1]:
                        run.append(mt)
                    else:
                        by_shape.setdefault(shape, []).append((gid, run))
                        run = [mt]
                by_shape.setdefault(shape, []).append((gid, run))
        for (r, c), runs in by_shape.items():
            views = [staged[gid][1][run[0].offset:run[0].offset + len(run) * r * c].view(len(run), r, c) for gid, run in runs]
            stack = views[0] if len(views) == 1 else torch.cat(views)
            O = self._orthogonalise(stack)
            sq = torch.linalg.vector_norm(O, dim=(-2, -1), dtype=torch.float32).square()
            i = 0
            for gid, run in runs:
                n = len(run)
                staged[gid][2][run[0].offset:run[0].offset + n * r * c].view(n, r, c).copy_(O[i:i + n])
                i += n
            idx = self._norm_idx_cache.get((r, c))
            if idx is None:
                idx = self._norm_idx_cache[(r, c)] = torch.tensor([mt.norm_idx for _, run in runs for mt in run],
                                                                  device=eng.device)
            u_sq.index_add_(0, idx, sq)
            del O, stack
        # 4. return the updates to the shards
        for gid, (g, u_full, o_full, _mine) in staged.items():
            if g.world > 1:
                tabs = self._transport_tables(g) if eng.symm is not None else None
                if tabs is not None:
                    o_shard = eng.symm.scatter_owned(g, o_full, tabs[1])
                elif eng.symm is not None:
                    o_shard = eng.symm.scatter_flat(g, o_full)
                else:
                    o_shard = torch.empty(g.shard_numel, dtype=cdt, device=eng.device)
                    du.reduce_scatter_sum(o_shard, o_full, group=g.group)
            else:
                o_shard = o_full
            out[gid] = o_shard
        return out

    # ------------------------------------------------------------------ checkpoint
    def zero_grad(self) -> None:
        self.engine.zero_grad()

    @torch.no_grad()
    def state_dict(self, rank0_only: bool = True) -> Dict:
        """Consolidated, world-size independent: per-parameter ``momentum`` / ``variance`` tensors."""
        eng = self.engine
        eng.reload_states()
        keep = (not rank0_only) or eng.mesh.rank == 0
        state: Dict[str, Dict[str, torch.Tensor]] = {}
        for g in eng.groups():
            gid = id(g)
            for key, store in (("momentum", self.m), ("variance", self.v)):
                if gid not in store:
                    continue
                full = eng._gather_master(store[gid], g)
                for s in g.specs:
                    t = eng.consolidate(s, g, full)       # whole tensors: tp slices reassembled, ep slabs concatenated
                    if keep:
                        state.setdefault(s.name, {})[key] = t.cpu().clone()
                del full
        extra = {}
        if self._xsq_cache is not None and self._xsq_version == getattr(eng, "master_version", 0):
            extra["muonh_sq_norms"] = self._xsq_cache.cpu()      # so that a resumed run keeps projecting onto the same spheres
        return {"state": state, "step": self.step_count, "algorithm": self.algorithm,
                "nadam_mu_product": self.nadam_mu_product, **extra} if keep else {}

    @torch.no_grad()
    def load_state_dict(self, sd: Dict) -> None:
        self.step_count = int(sd.get("step", 0))
        self.nadam_mu_product = float(sd.get("nadam_mu_product", 1.0))
        self._xsq_cache = None
        sq = sd.get("muonh_sq_norms")
        if sq is not None and sq.numel() == max(self.n_norm, 1):
            self._xsq_cache = sq.to(self.engine.device, torch.float32)
            self._xsq_version = getattr(self.engine, "master_version", 0)
        self.engine.reload_states()
        state = sd.get("state", {})
        for g in self.engine.groups():
            gid = id(g)
            for s, lo, hi, slo in g.local_slices():
                st = state.get(s.name)
                if not st:
                    continue
                for key, store in (("momentum", self.m), ("variance", self.v)):
                    if key in st and gid in store:
                        store[gid][slo:slo + hi - lo].copy_(self.engine.localize(s, g, st[key])[lo:hi].to(torch.float32))
