"""Tensor + sequence parallelism on two gloo ranks against the unsplit single-process model (fp32, AdamW)."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from archscale_b200 import Config
from archscale_b200.models.gpt import GPT, Block
from archscale_b200.ops import fused_linear_cross_entropy
from archscale_b200.optim.sharded import ShardedOptimizer
from archscale_b200.parallel import tp as tp_mod
from archscale_b200.parallel.fsdp import FSDPEngine
from archscale_b200.parallel.mesh import Mesh, build_mesh




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
    return Config.from_name("transformer_gqa4_d8", n_layer=2, ar=None, n_embd=128, n_head=4, n_query_groups=2, head_dim=32,
                            intermediate_size=256, vocab_size=512, padding_multiple=64, block_size=64, qk_norm=True)


def _model():
    torch.manual_seed(0)
    m = GPT(_cfg())
    m.reset_parameters()
    m.compute_dtype = torch.float32
    return m


def _data(steps):
    return torch.randint(0, 512, (steps, 2, 65), generator=torch.Generator().manual_seed(0))


def _run(m, mesh, steps):
    eng = FSDPEngine(m, mesh, unit_classes=(Block,), param_dtype=torch.float32)
    opt = ShardedOptimizer(eng, lr=1e-2, betas=(0.9, 0.95), algorithm="adamw", weight_decay=0.0)
    data = _data(steps)
    losses, norms = [], []
    for s in range(steps):
        batch = data[s]
        out = m(batch[:, :-1], use_flce_loss=True)
        tgt = batch[:, 1:]
        if mesh.tp > 1:
            tgt = tp_mod.token_slice(tgt, mesh.tp, mesh.tp_rank).contiguous()
        loss = fused_linear_cross_entropy(out.logits, out.weight, tgt)
        eng.backward(loss / mesh.tp)
        tp_mod.sync_replicated_grads(eng, mesh)
        norms.append(float(eng.clip_grad_norm_(1.0)))
        opt.step()
        opt.zero_grad()
        loss = loss.detach() / mesh.tp
        if mesh.tp > 1:
            dist.all_reduce(loss, group=mesh.tp_group)
        losses.append(float(loss))
    return losses, norms, eng


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        mesh = build_mesh(dp=1, tp=2)
        assert mesh.fsdp == 1 and mesh.tp == 2
        m = _model()
        tp_mod.apply_tensor_parallel(m, mesh)
        assert m.transformer.h[0].attn.q_proj.weight.shape == (64, 128)
        assert m.transformer.h[0].mlp.w1.weight.shape == (256, 128) and m.transformer.h[0].mlp.w3.weight.shape == (128, 128)
        losses, norms, _ = _run(m, mesh, 4)
        if rank == 0:
            q.put((losses, norms))
    finally:
        _leave_together()


def test_tp2_matches_single_process():
    ref_losses, ref_norms, _ = _run(_model(), Mesh(world=1, rank=0, dp=1, fsdp=1, tp=1), 4)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    losses, norms = q.get(timeout=300)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    for a, b in zip(losses, ref_losses):
        assert abs(a - b) < 2e-4 * max(1.0, abs(b)), (losses, ref_losses)
    for a, b in zip(norms, ref_norms):
        assert abs(a - b) < 2e-3 * max(1.0, abs(b)), (norms, ref_norms)
