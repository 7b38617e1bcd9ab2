"""Multi-GPU self-test of the peer-memory collectives against NCCL.  Launch one process per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        -m archscale_b200.parallel.selftest

Checks (rank 0 prints ``SELFTEST PASS`` / raises): pull all-gather == ``all_gather_into_tensor``
bitwise; pull reduce-scatter matches ``reduce_scatter_tensor`` in fp32; three training steps with
``fused_comm=True`` follow the NCCL run, also with two micro-steps per optimizer step (the heap gradient buffers
are then reused inside a step); prints bandwidths of both collectives.
"""
from __future__ import annotations

import os
import sys

import torch
import torch.distributed as dist


def _time(fn, iters=10):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def main() -> None:
    from archscale_b200.parallel import dist_utils as du
    from archscale_b200.parallel.symm import SymmetricHeap
    from archscale_b200.ops import backend

    du.init_process_group("nccl")
    rank, world = dist.get_rank(), dist.get_world_size()
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0)))
    ext = backend.require_extension()
    torch.manual_seed(rank)

    # ---- raw collectives
    S = 32 * 1024 * 1024                        # elements per shard
    heap = SymmetricHeap(dist.group.WORLD, S * 2 + S * world * 4 + (64 << 20), dev)
    off_lp = heap.alloc(S * 2)
    lp = heap.tensor(off_lp, (S,), torch.bfloat16)
    lp.copy_(torch.randn(S, device=dev))
    off_fg = heap.alloc(S * world * 4)
    fg = heap.tensor(off_fg, (S * world,), torch.float32)
    fg.copy_(torch.randn(S * world, device=dev))
    torch.cuda.synchronize()
    heap.barrier(0)
    full = torch.empty(S * world, dtype=torch.bfloat16, device=dev)
    ext.allgather_pull(heap.bases, off_lp, full, S * 2, rank, 32)
    ref = torch.empty_like(full)
    dist.all_gather_into_tensor(ref, lp)
    assert torch.equal(full, ref), "pull all-gather differs from NCCL"
    out = torch.empty(S, dtype=torch.float32, device=dev)
    ext.reduce_scatter_pull(heap.bases, off_fg, out, rank, 1.0 / world, False, 32)
    ref_rs = torch.empty_like(out)
    dist.reduce_scatter_tensor(ref_rs, fg.clone())
    ref_rs /= world
    err = float((out - ref_rs).abs().max())
    assert err < 1e-5, f"pull reduce-scatter error {err}"
    for ctas in (32, 64, 128, 296):
        t_ag = _time(lambda: ext.allgather_pull(heap.bases, off_lp, full, S * 2, rank, ctas))
        t_rs = _time(lambda: ext.reduce_scatter_pull(heap.bases, off_fg, out, rank, 1.0 / world, False, ctas))
        if rank == 0:
            print(f"ctas={ctas}: pull all-gather {S * 2 * (world - 1) / t_ag / 1e6:.0f} GB/s in ({t_ag:.3f} ms); "
                  f"pull reduce-scatter {S * 4 * (world - 1) / t_rs / 1e6:.0f} GB/s in ({t_rs:.3f} ms)", flush=True)
    t_ag = _time(lambda: dist.all_gather_into_tensor(ref, lp))
    t_rs = _time(lambda: dist.reduce_scatter_tensor(ref_rs, fg))
    if rank == 0:
        print(f"NCCL: all-gather {S * 2 * (world - 1) / t_ag / 1e6:.0f} GB/s ({t_ag:.3f} ms); reduce-scatter "
              f"{S * 4 * (world - 1) / t_rs / 1e6:.0f} GB/s ({t_rs:.3f} ms)", flush=True)

    # ---- all-gather fused into the consuming GEMM
    N, K, M = 2048, 2048, 32768
    shard_elems = 6 * 1024 * 1024                       # per-rank shard of a "unit" (bf16)
    off_w = heap.alloc(shard_elems * 2)
    wshard = heap.tensor(off_w, (shard_elems,), torch.bfloat16)
    wshard.copy_(torch.randn(shard_elems, device=dev) * 0.02)
    torch.cuda.synchronize()
    heap.barrier(0)
    gathered = torch.zeros(shard_elems * world, dtype=torch.bfloat16, device=dev)
    flags = torch.zeros((shard_elems * world * 2 + 262143) // 262144, dtype=torch.int32, device=dev)
    x = (torch.randn(M, K, device=dev) * 0.1).bfloat16()
    y = ext.ag_gemm(x, heap.bases, off_w, gathered, shard_elems * 2, 0, N, flags, 1, rank, 16)
    ref_full = torch.empty_like(gathered)
    dist.all_gather_into_tensor(ref_full, wshard)
    assert torch.equal(gathered, ref_full), "fused gather produced a different buffer"
    y_ref = x.float() @ ref_full[: N * K].view(N, K).float().t()
    rel = float((y.float() - y_ref).norm() / y_ref.norm())
    assert rel < 1e-2, f"ag_gemm result off by {rel}"
    ep = [1]

    def fused():
        ep[0] += 1
        ext.ag_gemm(x, heap.bases, off_w, gathered, shard_elems * 2, 0, N, flags, ep[0], rank, 16)

    def separate():
        ext.allgather_pull(heap.bases, off_w, gathered, shard_elems * 2, rank, 48)
        ext.gemm_bf16(x, gathered[: N * K].view(N, K), 0, torch.bfloat16, None)

    def nccl_sep():
        dist.all_gather_into_tensor(ref_full, wshard)
        x @ ref_full[: N * K].view(N, K).t()

    t_f, t_s, t_n = _time(fused), _time(separate), _time(nccl_sep)
    t_g = _time(lambda: ext.gemm_bf16(x, gathered[: N * K].view(N, K), 0, torch.bfloat16, None))
    if rank == 0:
        fl = 2.0 * M * N * K
        nv = shard_elems * 2 * (world - 1)
        print(f"ag_gemm fused {t_f:.3f} ms | pull-gather then gemm {t_s:.3f} ms | NCCL gather then cuBLAS {t_n:.3f} ms | "
              f"gemm alone {t_g:.3f} ms; roofline max(flops/peak, bytes/link) = "
              f"{max(fl / 1.7138e15, nv / 770e9) * 1e3:.3f} ms → fraction {max(fl / 1.7138e15, nv / 770e9) * 1e3 / t_f:.2f}",
              flush=True)

    # ---- training steps: fused vs NCCL
    from archscale_b200 import Config
    from archscale_b200.models.gpt import GPT, Block
    from archscale_b200.ops import fused_linear_cross_entropy
    from archscale_b200.optim.sharded import ShardedOptimizer
    from archscale_b200.parallel.fsdp import FSDPEngine
    from archscale_b200.parallel.mesh import build_mesh

    mesh = build_mesh()

    def run(fused: bool, accum: int = 1):
        torch.manual_seed(0)
        cfg = Config.from_name("transformer_gqa4_d16", n_layer=4, ar=None, n_embd=1024, n_head=8, n_query_groups=4,
                               head_dim=128, intermediate_size=2816, block_size=1024, qk_norm=True, mup=True,
                               depth_scale=True, use_muon=True, use_muonh=True, head_init_std=0.02)
        with torch.device(dev):
            model = GPT(cfg)
        model.reset_parameters()
        eng = FSDPEngine(model, mesh, unit_classes=(Block,), param_dtype=torch.bfloat16, device=dev, fused_comm=fused)
        opt = ShardedOptimizer(eng, lr=2e-3, algorithm="muonh")
        g = torch.Generator().manual_seed(100 + rank)
        losses = []
        for _ in range(4):
            for _micro in range(accum):      # accum > 1: the heap gradient buffers are reused inside one optimizer step
                data = torch.randint(0, cfg.vocab_size, (2, 1025), generator=g).to(dev)
                o = model(data[:, :-1], use_flce_loss=True)
                loss = fused_linear_cross_entropy(o.logits, o.weight, data[:, 1:])
                eng.backward(loss / accum)
            eng.clip_grad_norm_(1.0)
            opt.step()
            opt.zero_grad()
            l = loss.detach().clone()
            dist.all_reduce(l)
            losses.append(float(l) / world)
        return losses

    a = run(False)
    b = run(True)
    torch.cuda.synchronize()
    status = ext.device_status()
    if rank == 0:
        print("NCCL  losses", a)
        print("fused losses", b, "device status", status, flush=True)
    assert status == 0, f"device status {status}"
    for x, y in zip(a, b):
        assert abs(x - y) < 5e-2, (a, b)
    a2, b2 = run(False, accum=2), run(True, accum=2)
    torch.cuda.synchronize()
    status = ext.device_status()
    if rank == 0:
        print("gradient accumulation 2: NCCL", a2, "fused", b2, "device status", status, flush=True)
    assert status == 0, f"device status {status}"
    for x, y in zip(a2, b2):
        assert abs(x - y) < 5e-2, (a2, b2)
    dist.barrier()
    if rank == 0:
        print("SELFTEST PASS", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
