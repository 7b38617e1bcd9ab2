"""MuonBall: one step against a dense restatement, and sharded (2 gloo ranks) against single process."""
import math
import os

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from archscale_b200 import Config
from archscale_b200.models.gpt import GPT, Block
from archscale_b200.ops import fused_linear_cross_entropy
from archscale_b200.ops.newton_schulz import POLAR_EXPRESS_COEFFS, newton_schulz_ref
from archscale_b200.optim.muon_ball import ShardedMuonBall, power_iteration
from archscale_b200.parallel.fsdp import FSDPEngine
from archscale_b200.parallel.mesh import build_mesh




def _leave_together():
    """Ranks leave the process group together: a rank that closes its sockets while a peer is still inside its last
    collective's teardown can abort that peer."""
    import datetime
    try:
        dist.monitored_barrier(timeout=datetime.timedelta(seconds=30))
    except Exception:
        pass
    dist.destroy_process_group()

def _free_port() -> int:
    import socket
    with socket.socket() as sk:
        sk.bind(("127.0.0.1", 0))
        return sk.getsockname()[1]

def _cfg():
    return Config.from_name("transformer_gqa4_d8", n_layer=2, ar=None, n_embd=128, n_head=2, n_query_groups=1, head_dim=64,
                            intermediate_size=256, vocab_size=512, padding_multiple=64, block_size=64)


def _build():
    torch.manual_seed(0)
    m = GPT(_cfg())
    m.reset_parameters()
    m.compute_dtype = torch.float32
    eng = FSDPEngine(m, build_mesh(), unit_classes=(Block,), param_dtype=torch.float32)
    opt = ShardedMuonBall(eng, lr=0.02, betas=(0.9, 0.95), mu=0.95)
    return m, eng, opt


def _step(m, eng, opt, batch):
    out = m(batch[:, :-1], use_flce_loss=True)
    loss = fused_linear_cross_entropy(out.logits, out.weight, batch[:, 1:])
    eng.backward(loss)
    opt.step()
    opt.zero_grad()
    return float(loss)


def test_power_iteration_matches_svd():
    torch.manual_seed(1)
    w = torch.randn(3, 48, 80)
    s = power_iteration(w, 200)
    ref = torch.linalg.svdvals(w)[:, 0]
    assert torch.allclose(s, ref, rtol=1e-3)


def _master(eng, suffix, what="master"):
    for grp in eng.groups():
        for s in grp.specs:
            if s.name.endswith(suffix):
                return getattr(grp, what)[s.offset:s.offset + s.numel].view(s.shape).clone()
    raise KeyError(suffix)


def test_one_step_matches_dense_restatement():
    m, eng, opt = _build()
    w0 = _master(eng, "h.0.mlp.w3.weight")
    batch = torch.randint(0, 512, (2, 65), generator=torch.Generator().manual_seed(0))
    out = m(batch[:, :-1], use_flce_loss=True)
    loss = fused_linear_cross_entropy(out.logits, out.weight, batch[:, 1:])
    eng.backward(loss)
    g = _master(eng, "h.0.mlp.w3.weight", "grad")
    opt.step()
    rows, cols = w0.shape
    sigma = torch.linalg.svdvals(w0)[0]
    w = w0 * (math.sqrt(rows / cols) / (sigma + 1e-8))
    mom = g.clone()                                   # first step: M = g, Nesterov: g + mu·M
    u = g + 0.95 * mom
    coeffs = [POLAR_EXPRESS_COEFFS[i] for i in range(5)]
    phi = newton_schulz_ref(u, 1e-7, coeffs=coeffs).float()
    w = w - 0.02 * math.sqrt(rows / cols) * phi
    got = _master(eng, "h.0.mlp.w3.weight")
    assert (got - w).abs().max() < 2e-3 * w.abs().max(), (got - w).abs().max()
    assert abs(float(opt.last_sigma.max()) - float(torch.linalg.svdvals(w0)[0])) < 0.5


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        m, eng, opt = _build()
        data = torch.randint(0, 512, (3, 4, 65), generator=torch.Generator().manual_seed(0))
        losses = []
        for s in range(3):
            l = torch.tensor(_step(m, eng, opt, data[s, rank * 2:(rank + 1) * 2]))
            dist.all_reduce(l)
            losses.append(float(l) / world)
        if rank == 0:
            q.put(losses)
    finally:
        _leave_together()


def test_two_ranks_match_single_process():
    m, eng, opt = _build()
    data = torch.randint(0, 512, (3, 4, 65), generator=torch.Generator().manual_seed(0))
    ref = [_step(m, eng, opt, data[s]) for s in range(3)]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = q.get(timeout=300)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    for a, b in zip(got, ref):
        assert abs(a - b) < 5e-3 * max(1.0, abs(b)), (got, ref)
