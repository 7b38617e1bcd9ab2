"""Multi-GPU self-test of expert parallelism: peer-memory dispatch/combine vs the all_to_all baseline.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        -m archscale_b200.parallel.selftest_ep
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist


def main() -> None:
    from archscale_b200.ops import backend, router_topk_softmax
    from archscale_b200.parallel import dist_utils as du
    from archscale_b200.parallel import ep

    du.init_process_group("nccl")
    rank, world = dist.get_rank(), dist.get_world_size()
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0)))
    ext = backend.require_extension()
    N, C, E, I, K = 4096, 1024, 64, 256, 8
    el = E // world
    g = torch.Generator(device="cpu").manual_seed(7)
    w_in_all = (torch.randn(E, 2 * I, C, generator=g) * 0.03)
    w_out_all = (torch.randn(E, C, I, generator=g) * 0.03)
    torch.manual_seed(100 + rank)

    def run(peer: bool):
        ep.USE_PEER_TRANSPORT = peer
        torch.manual_seed(100 + rank)
        x = (torch.randn(N, C, device=dev) * 0.5).bfloat16().requires_grad_()
        wi = w_in_all[rank * el:(rank + 1) * el].to(dev).bfloat16().requires_grad_()
        wo = w_out_all[rank * el:(rank + 1) * el].to(dev).bfloat16().requires_grad_()
        lg = torch.randn(N, E, device=dev, requires_grad=True)
        sc, idx = router_topk_softmax(lg, K, sqrt_gate=True)
        out = ep.moe_ffn_expert_parallel(x, wi, wo, sc, idx, E, dist.group.WORLD)
        gout = torch.randn(N, C, device=dev, generator=torch.Generator(device=dev).manual_seed(5 + rank)).bfloat16()
        out.backward(gout)
        return [t.detach().float() for t in (out, x.grad, wi.grad, wo.grad, lg.grad)]

    a = run(False)
    b = run(True)
    torch.cuda.synchronize()
    assert ext.device_status() == 0, ext.device_status()
    names = ("out", "dx", "dw_in", "dw_out", "dlogits")
    for n, x, y in zip(names, a, b):
        rel = float((x - y).norm() / (x.norm() + 1e-12))
        if rank == 0:
            print(f"{n}: rel diff peer vs all_to_all = {rel:.2e}", flush=True)
        assert rel < 2e-2, (n, rel)

    def timeit(peer):
        ep.USE_PEER_TRANSPORT = peer
        x = (torch.randn(16384, C, device=dev) * 0.5).bfloat16().requires_grad_()
        wi = w_in_all[rank * el:(rank + 1) * el].to(dev).bfloat16().requires_grad_()
        wo = w_out_all[rank * el:(rank + 1) * el].to(dev).bfloat16().requires_grad_()
        lg = torch.randn(16384, E, device=dev)
        sc, idx = router_topk_softmax(lg, K, sqrt_gate=True)

        def step():
            out = ep.moe_ffn_expert_parallel(x, wi, wo, sc, idx, E, dist.group.WORLD)
            out.backward(torch.ones_like(out))
        for _ in range(3):
            step()
        torch.cuda.synchronize(); dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(5):
            step()
        e1.record(); torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / 5], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    t_a, t_p = timeit(False), timeit(True)
    if rank == 0:
        print(f"MoE layer fwd+bwd, 16384 tokens/rank, E=64 top-8: all_to_all {t_a:.3f} ms, peer pulls {t_p:.3f} ms", flush=True)
        print("SELFTEST EP PASS", flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
