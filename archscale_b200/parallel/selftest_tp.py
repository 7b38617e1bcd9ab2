"""Multi-GPU self-test of the fused tensor-parallel layers: all-gather→GEMM and GEMM→reduce-scatter over peer memory
against NCCL collectives + the plain GEMM, numerics and device-timed speed (max over ranks).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        -m archscale_b200.parallel.selftest_tp
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist


def main() -> None:
    from archscale_b200.ops import backend
    from archscale_b200.ops.gemm import matmul_nt
    from archscale_b200.parallel import dist_utils as du
    from archscale_b200.parallel import tp
    from archscale_b200.parallel.mesh import build_mesh

    du.init_process_group("nccl")
    rank, world = dist.get_rank(), dist.get_world_size()
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0)))
    torch.cuda.set_device(dev)
    ext = backend.require_extension()
    mesh = build_mesh(dp=1, tp=world)
    M, C, I = 32768, 2048, 5632                      # tokens of one micro-batch, d_model, MLP width (d16 shapes)
    n = M // world
    ctx = tp.FusedTPContext(mesh, dev, max_tokens=M, max_features=C)
    torch.manual_seed(10 + rank)
    x_local = (torch.randn(n, C, device=dev) * 0.5).bfloat16()
    w1 = (torch.randn(2 * I // world, C, device=dev) * 0.02).bfloat16()          # column-parallel shard
    a = (torch.randn(M, I // world, device=dev) * 0.5).bfloat16()               # row-parallel input
    w3 = (torch.randn(C, I // world, device=dev) * 0.02).bfloat16()

    def ref_ag():
        full = torch.empty(M, C, device=dev, dtype=torch.bfloat16)
        dist.all_gather_into_tensor(full, x_local)
        return full, matmul_nt(full, w1)

    def ref_rs():
        part = matmul_nt(a, w3)
        out = torch.empty(n, C, device=dev, dtype=torch.bfloat16)
        dist.reduce_scatter_tensor(out, part)
        return out

    for it in range(3):                              # three rounds: both buffer parities and counter accumulation
        xf, y = ctx.ag_linear(x_local, w1)
        xr, yr = ref_ag()
        assert torch.equal(xf, xr), "gathered activations differ"
        rel = float((y.float() - yr.float()).norm() / yr.float().norm())
        assert rel < 1e-3, ("ag_linear", it, rel)
        o = ctx.linear_rs(a, w3)
        orf = ref_rs()
        rel2 = float((o.float() - orf.float()).norm() / orf.float().norm())
        assert rel2 < 1e-2, ("linear_rs", it, rel2)
    torch.cuda.synchronize()
    assert ext.device_status() == 0, ext.device_status()
    if rank == 0:
        print(f"numerics ok: ag_linear rel {rel:.1e}, linear_rs rel {rel2:.1e}", flush=True)

    def timed(fn, iters=10):
        for _ in range(3):
            fn()
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / iters], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    t_ag_f, t_ag_n = timed(lambda: ctx.ag_linear(x_local, w1)), timed(ref_ag)
    t_rs_f, t_rs_n = timed(lambda: ctx.linear_rs(a, w3)), timed(ref_rs)
    t_g1 = timed(lambda: matmul_nt(torch.empty(M, C, device=dev, dtype=torch.bfloat16), w1))
    t_g3 = timed(lambda: matmul_nt(a, w3))
    fl1, fl3 = 2.0 * M * (2 * I // world) * C, 2.0 * M * C * (I // world)
    link = 770e9
    roof_ag = max(fl1 / 1.7138e15, (world - 1) * n * C * 2 / link) * 1e3
    roof_rs = max(fl3 / 1.7138e15, (world - 1) * n * C * 2 / link) * 1e3
    if rank == 0:
        print(f"all-gather→GEMM  fused {t_ag_f:.3f} ms | NCCL all-gather + GEMM {t_ag_n:.3f} ms | GEMM alone {t_g1:.3f} ms | "
              f"roofline {roof_ag:.3f} ms ({roof_ag / t_ag_f:.2f} of roofline)", flush=True)
        print(f"GEMM→reduce-scatter fused {t_rs_f:.3f} ms | GEMM + NCCL reduce-scatter {t_rs_n:.3f} ms | GEMM alone {t_g3:.3f} ms | "
              f"roofline {roof_rs:.3f} ms ({roof_rs / t_rs_f:.2f} of roofline)", flush=True)
    torch.cuda.synchronize()
    assert ext.device_status() == 0, ext.device_status()
    dist.barrier()
    if rank == 0:
        print("selftest_tp PASS", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
