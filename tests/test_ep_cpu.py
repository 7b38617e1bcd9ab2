"""Expert-parallel MoE over gloo ranks equals the single-process oracle (forward and gradients)."""
import os

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from archscale_b200.ops.moe import moe_ffn_ref, router_topk_softmax_ref
from archscale_b200.parallel.ep import moe_ffn_expert_parallel



def _leave_together():
    """Ranks leave the process group together: a rank that closes its sockets while a peer is still inside its last
    collective's teardown can abort that peer."""
    import datetime
    try:
        dist.monitored_barrier(timeout=datetime.timedelta(seconds=30))
    except Exception:
        pass
    dist.destroy_process_group()

def _make(world, N=24, C=16, E=8, I=8, K=2):
    g = torch.Generator().manual_seed(0)
    x = torch.randn(world, N, C, generator=g)
    w_in = torch.randn(E, 2 * I, C, generator=g) * 0.3
    w_out = torch.randn(E, C, I, generator=g) * 0.3
    logits = torch.randn(world, N, E, generator=g)
    gout = torch.randn(world, N, C, generator=g)
    return x, w_in, w_out, logits, gout, K


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        x, w_in, w_out, logits, gout, K = _make(world)
        E = w_in.shape[0]
        el = E // world
        xr = x[rank].clone().requires_grad_()
        wi = w_in[rank * el:(rank + 1) * el].clone().requires_grad_()
        wo = w_out[rank * el:(rank + 1) * el].clone().requires_grad_()
        lg = logits[rank].clone().requires_grad_()
        scores, idx = router_topk_softmax_ref(lg, K, sqrt_gate=True)
        out = moe_ffn_expert_parallel(xr, wi, wo, scores, idx, E, dist.group.WORLD)
        out.backward(gout[rank])
        q.put((rank, out.detach(), xr.grad, wi.grad, wo.grad, lg.grad))
    finally:
        _leave_together()


def test_expert_parallel_matches_oracle():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.SimpleQueue()
    procs = [ctx.Process(target=_worker, args=(r, world, 29631, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = {}
    for _ in range(world):
        r = q.get()
        results[r[0]] = [t.clone() for t in r[1:]]
    for p in procs:
        p.join()
        assert p.exitcode == 0
    x, w_in, w_out, logits, gout, K = _make(world)
    E = w_in.shape[0]
    el = E // world
    wi, wo = w_in.clone().requires_grad_(), w_out.clone().requires_grad_()
    for rank in range(world):
        xr, lg = x[rank].clone().requires_grad_(), logits[rank].clone().requires_grad_()
        scores, idx = router_topk_softmax_ref(lg, K, sqrt_gate=True)
        ref = moe_ffn_ref(xr, wi, wo, scores, idx)
        ref.backward(gout[rank])
        out, gx, gwi, gwo, glg = results[rank]
        assert torch.allclose(out, ref.detach(), atol=1e-5)
        assert torch.allclose(gx, xr.grad, atol=1e-5)
        assert torch.allclose(glg, lg.grad, atol=1e-5)
    for rank in range(world):
        _, _, gwi, gwo, _ = results[rank]
        assert torch.allclose(gwi, wi.grad[rank * el:(rank + 1) * el], atol=1e-5)     # sums over all ranks' tokens
        assert torch.allclose(gwo, wo.grad[rank * el:(rank + 1) * el], atol=1e-5)
