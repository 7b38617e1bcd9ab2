"""MuonBall on sharded parameters: Muon with the weights kept on a spectral sphere.

Per 2-D hidden matrix ``W`` (out × in) and step (the algorithm of
`emerging_optimizers/orthogonalized_optimizers/muon_ball.py:60-142,325-347`, selected by ``muonball`` in the
train name, `pretrain.py:655-683`):

1. ``σ`` = leading singular value of ``W`` by bilateral power iteration (50 steps);
2. hard retraction ``W ← (R / σ)·W`` with ``R = sqrt(out / in)`` (``radius_mode="spectral_mup"``);
3. ``Φ = msign(M)`` for the Nesterov momentum ``M``: five matrix-sign iterations with the Polar-Express coefficients;
4. ``W ← W − lr·sqrt(out / in)·Φ`` (``scale_mode="spectral_mup"``), no weight decay.

Vectors, embeddings and the head take AdamW.  Everything that is shared with Muon — momentum on the local shard,
assembling whole matrices on an owner rank, the three batched tcgen05 GEMMs per iteration, returning the update to
the shards — is inherited from :class:`ShardedOptimizer`; this class adds the retraction pass (one extra gather of
the bf16 weights, one all-reduce of the per-matrix scales) and swaps the coefficient schedule.
"""
from __future__ import annotations

import math
from typing import Dict, List, Tuple

import torch

from archscale_b200 import ops
from archscale_b200.ops.newton_schulz import POLAR_EXPRESS_COEFFS
from archscale_b200.optim.sharded import ShardedOptimizer, _Mat
from archscale_b200.parallel import dist_utils as du


@torch.no_grad()
def power_iteration(w: torch.Tensor, steps: int = 50) -> torch.Tensor:
    """Leading singular value of every matrix of ``w`` (..., rows, cols)
    (`spectral_ball_utils.py:151-166`: start from the all-ones vector, alternate ``WᵀW v`` and normalise)."""
    v = torch.ones_like(w[..., :1, :]).transpose(-2, -1)
    for _ in range(steps):
        v = torch.nn.functional.normalize(w.transpose(-2, -1) @ (w @ v), dim=-2)
    u = torch.nn.functional.normalize(w @ v, dim=-2)
    return (u.transpose(-2, -1) @ w @ v).squeeze(-1).squeeze(-1).float()


class ShardedMuonBall(ShardedOptimizer):
    def __init__(self, engine, lr: float = 1e-3, betas: Tuple[float, float] = (0.9, 0.95), eps: float = 1e-8,
                 vector_weight_decay: float = 0.0, mu: float = 0.95, power_iteration_steps: int = 50, msign_steps: int = 5,
                 **kw) -> None:
        super().__init__(engine, lr=lr, betas=betas, eps=eps, weight_decay=0.0, vector_weight_decay=vector_weight_decay,
                         weight_lr_mult=1.0, algorithm="muon", mu=mu, nesterov=True, adjust_lr="spectral_norm",
                         ns_epsilon=1e-7, **kw)
        self.power_iteration_steps, self.msign_steps = power_iteration_steps, msign_steps
        self.last_sigma: torch.Tensor = torch.zeros(0)

    def _orthogonalise(self, stack: torch.Tensor) -> torch.Tensor:
        coeffs = [POLAR_EXPRESS_COEFFS[min(i, len(POLAR_EXPRESS_COEFFS) - 1)] for i in range(self.msign_steps)]
        return ops.newton_schulz(stack, epsilon=1e-7, coeffs=coeffs)

    @torch.no_grad()
    def _retract(self) -> None:
        """Scale every Muon matrix onto its spectral sphere: owners measure σ on the gathered bf16 weights, the
        per-matrix factors R/σ are shared with one all-reduce, every rank scales its slice of the fp32 master."""
        eng = self.engine
        dev = eng.device
        cdt = torch.bfloat16 if eng.is_cuda else torch.float32
        scale = torch.zeros(max(self.n_norm, 1), dtype=torch.float32, device=dev)
        sigma = torch.zeros_like(scale)
        groups = {id(mt.group): mt.group for mt in self.mats}
        for gid, g in groups.items():
            if g.world > 1:
                w_full = torch.empty(g.padded, dtype=cdt, device=dev)
                du.all_gather_into(w_full, g.master.to(cdt), group=g.group)
            else:
                w_full = g.master.to(cdt)
            by_shape: Dict[Tuple[int, int], List[_Mat]] = {}
            for mt in self.mats:
                if mt.group is g and mt.owner == g.rank:
                    by_shape.setdefault((mt.rows, mt.cols), []).append(mt)
            for (r, c), lst in by_shape.items():
                stack = torch.stack([w_full[mt.offset:mt.offset + r * c].view(r, c) for mt in lst])
                s = power_iteration(stack, self.power_iteration_steps)
                idx = torch.tensor([mt.norm_idx for mt in lst], device=dev)
                sigma[idx] = s
                scale[idx] = math.sqrt(r / c) / (s.clamp_min(0.0) + 1e-8)
        if eng.mesh.fsdp > 1:
            packed = torch.stack((scale, sigma))
            keep = packed[:, self.local_norm_idx].clone() if self.local_norm_idx is not None else None
            du.all_reduce_sum(packed, group=eng.mesh.fsdp_group)
            if keep is not None:
                packed[:, self.local_norm_idx] = keep
            scale, sigma = packed[0], packed[1]
        self.last_sigma = sigma
        xs, ks = [], []
        for mt in self.mats:
            g = mt.group
            a, b = g.shard_range()
            lo, hi = max(mt.offset, a), min(mt.offset + mt.rows * mt.cols, b)
            if lo < hi:
                xs.append(g.master[lo - a:hi - a])
                ks.append(mt.norm_idx)
        if xs:
            torch._foreach_mul_(xs, list(scale[torch.tensor(ks, device=dev)].unbind(0)))

    @torch.no_grad()
    def step(self, lr=None, weight_decay=None, **kw) -> None:
        self._retract()
        super().step(lr=lr, weight_decay=0.0, **kw)
