"""Device mesh with named axes ``dp`` (replicate) × ``fsdp`` (shard) × ``tp`` (tensor parallel);
expert parallelism re-uses ranks of ``fsdp`` (``ep`` axis is a view of the same ranks).

The reference builds a 2-D ``(data_parallel, tensor_parallel)`` mesh through Lightning Fabric
where "tensor_parallel" is really the intra-node FSDP shard axis (`pretrain.py:384-387`).  Here
the axes are named for what they do.  Rank order: ``rank = (dp_i · fsdp + fsdp_i) · tp + tp_i``
so tensor-parallel peers are adjacent GPUs.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch.distributed as dist

from . import dist_utils as du


@dataclass
class Mesh:
    world: int
    rank: int
    dp: int
    fsdp: int
    tp: int
    dp_group: Optional[object] = None
    fsdp_group: Optional[object] = None
    tp_group: Optional[object] = None
    ep: int = 1
    ep_group: Optional[object] = None

    @property
    def dp_rank(self) -> int:
        return self.rank // (self.fsdp * self.tp)

    @property
    def fsdp_rank(self) -> int:
        return (self.rank // self.tp) % self.fsdp

    @property
    def tp_rank(self) -> int:
        return self.rank % self.tp

    @property
    def ep_rank(self) -> int:
        return self.fsdp_rank % self.ep

    @property
    def data_rank(self) -> int:
        """Index of this rank among ranks that read different data (tp peers share a batch)."""
        return self.rank // self.tp

    @property
    def data_world(self) -> int:
        return self.dp * self.fsdp


def build_mesh(dp: int = 1, tp: int = 1, ep: int = 1) -> Mesh:
    w, r = du.world_size(), du.rank()
    assert w % (dp * tp) == 0, f"world {w} not divisible by dp*tp = {dp * tp}"
    fsdp = w // (dp * tp)
    m = Mesh(world=w, rank=r, dp=dp, fsdp=fsdp, tp=tp, ep=ep)
    if w == 1:
        return m

    def groups(make_ranks):
        mine = None
        seen = set()
        for rr in range(w):
            ranks = tuple(make_ranks(rr))
            if ranks in seen:
                continue
            seen.add(ranks)
            g = dist.new_group(list(ranks)) if len(ranks) > 1 and len(ranks) < w else (dist.group.WORLD if len(ranks) == w else None)
            if r in ranks:
                mine = g
        return mine

    idx = lambda d, f, t: (d * fsdp + f) * tp + t
    coords = lambda rr: (rr // (fsdp * tp), (rr // tp) % fsdp, rr % tp)
    m.tp_group = groups(lambda rr: [idx(coords(rr)[0], coords(rr)[1], t) for t in range(tp)])
    m.fsdp_group = groups(lambda rr: [idx(coords(rr)[0], f, coords(rr)[2]) for f in range(fsdp)])
    m.dp_group = groups(lambda rr: [idx(d, coords(rr)[1], coords(rr)[2]) for d in range(dp)])
    if ep > 1:
        assert fsdp % ep == 0, "ep must divide the fsdp axis"
        if ep == fsdp:
            m.ep_group = m.fsdp_group
        else:
            m.ep_group = groups(lambda rr: [idx(coords(rr)[0], (coords(rr)[1] // ep) * ep + e, coords(rr)[2])
                                            for e in range(ep)])
    return m
