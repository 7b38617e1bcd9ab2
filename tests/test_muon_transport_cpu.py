"""Owner-only Muon transport: the piece tables (which 16-byte ranges a rank pulls from which peer) reproduce, when replayed
on the host, what the full all-gather / reduce-scatter transport delivers: every owner sees its whole matrices, every shard
gets the orthogonalised values of exactly its range."""
from types import SimpleNamespace

import torch

from archscale_b200.optim.sharded import ShardedOptimizer, _Mat
from archscale_b200.parallel.symm import SymmetricContext


def _tables(world, S, mats_spec, matrix_numel):
    out = []
    for r in range(world):
        g = SimpleNamespace(shard_numel=S, rank=r, world=world, matrix_numel=matrix_numel)
        mats = []
        for off, rows, cols, owner in mats_spec:
            mt = _Mat.__new__(_Mat)
            mt.group, mt.offset, mt.rows, mt.cols, mt.owner = g, off, rows, cols, owner
            mats.append(mt)
        fake = SimpleNamespace(mats=mats, engine=SimpleNamespace(symm=SymmetricContext, device=torch.device("cpu")))
        out.append(ShardedOptimizer._transport_tables(fake, g))
    return out


def _replay(table, sources, dst):
    for src, d, packed in table.tolist():
        n, rank = packed & 0xffffffff, packed >> 32
        assert n <= 4096
        dst[d * 8:(d + n) * 8] = sources[rank][src * 8:(src + n) * 8]


def test_owner_only_transport_equals_full_gather():
    world, S = 4, 4096 * 3                      # shards of 12288 elements
    # matrices back to back from offset 0, spanning shard boundaries; owners round-robin
    shapes = [(64, 128), (128, 64), (96, 128), (8, 1024), (160, 64)]
    specs, off = [], 0
    for i, (r, c) in enumerate(shapes):
        specs.append((off, r, c, i % world))
        off += r * c
    matrix_numel = off
    assert matrix_numel <= world * S
    tabs = _tables(world, S, specs, matrix_numel)
    assert all(t is not None for t in tabs)
    flat_u = torch.arange(world * S, dtype=torch.float32)
    shards = [flat_u[r * S:(r + 1) * S] for r in range(world)]
    # gather: owner r must see its matrices whole
    o_bufs = []
    for r in range(world):
        full = torch.full((world * S,), -1.0)
        _replay(tabs[r][0], shards, full)
        ob = torch.full((world * S,), -7.0)      # owners' O buffers: garbage outside the owned ranges
        for off_, rows, cols, owner in specs:
            if owner == r:
                assert torch.equal(full[off_:off_ + rows * cols], flat_u[off_:off_ + rows * cols])
                ob[off_:off_ + rows * cols] = 2 * flat_u[off_:off_ + rows * cols]      # "orthogonalised"
        o_bufs.append(ob)
    # return: shard r gets 2·u on its part of the matrix range, from the right owners only
    for r in range(world):
        out = torch.full((S,), -3.0)
        _replay(tabs[r][1], o_bufs, out)
        a, b = r * S, min((r + 1) * S, matrix_numel)
        if b > a:
            assert torch.equal(out[:b - a], 2 * flat_u[a:b])


def test_unaligned_ranges_fall_back():
    tabs = _tables(2, 1000, [(0, 10, 10, 0), (100, 30, 30, 1)], 1000)     # offsets / sizes not multiples of 8
    assert tabs[0] is None and tabs[1] is None
