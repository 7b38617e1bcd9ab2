"""CPU / gloo tests of the sharding engine, the hybrid optimizer and checkpoint round-trip.

The main case is the plumbing configuration of the benchmark spec: a 2-layer dense GQA transformer
(d_model 256, 2 query heads / 1 KV head, head_dim 128, SwiGLU 1024, vocab 32000, untied) in fp32 on two
gloo ranks, Muon (5 Newton–Schulz iterations, momentum 0.95) on hidden matrices + AdamW (lr 1e-3, betas
0.9/0.95) on embeddings and norms, micro-batch 2×512 of uniform-random tokens (seed 0): 10 steps, save,
reload, and the loss of step 11 must be bitwise identical to the uninterrupted run.
"""
import os
import tempfile

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from archscale_b200 import Config
from archscale_b200.models.gpt import GPT, Block
from archscale_b200.ops import fused_linear_cross_entropy
from archscale_b200.optim.sharded import ShardedOptimizer
from archscale_b200.parallel.fsdp import FSDPEngine
from archscale_b200.parallel.mesh import build_mesh
from archscale_b200.utils import checkpoint as ckpt



def _leave_together():
    """Ranks leave the process group together: a rank that closes its sockets while a peer is still inside its last
    collective's teardown can abort that peer."""
    import datetime
    try:
        dist.monitored_barrier(timeout=datetime.timedelta(seconds=30))
    except Exception:
        pass
    dist.destroy_process_group()

def _cfg(**kw):
    base = dict(n_layer=2, ar=None, n_embd=256, n_head=2, n_query_groups=1, head_dim=128, intermediate_size=1024,
                vocab_size=32000, padding_multiple=64, block_size=512, rope_base=10000, norm_eps=1e-5)
    base.update(kw)
    return Config.from_name("transformer_gqa4_d8", **base)


def _build(cfg, algo, lr=1e-3):
    torch.manual_seed(0)
    m = GPT(cfg)
    m.reset_parameters()
    m.compute_dtype = torch.float32
    eng = FSDPEngine(m, build_mesh(), unit_classes=(Block,), param_dtype=torch.float32)
    opt = ShardedOptimizer(eng, lr=lr, betas=(0.9, 0.95), algorithm=algo, mu=0.95, nesterov=True, weight_decay=0.0)
    return m, eng, opt


def _step(m, eng, opt, batch):
    out = m(batch[:, :-1], use_flce_loss=True)
    loss = fused_linear_cross_entropy(out.logits, out.weight, batch[:, 1:])
    eng.backward(loss)
    eng.clip_grad_norm_(1.0)
    opt.step()
    opt.zero_grad()
    return loss.detach().clone()


def _data(world, steps, per_rank=2, T=512):
    g = torch.Generator().manual_seed(0)
    return torch.randint(0, 32000, (steps, world * per_rank, T + 1), generator=g)


def _worker(rank, world, port, tmp, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        data = _data(world, 11)
        mine = lambda s: data[s, rank * 2:(rank + 1) * 2]
        m, eng, opt = _build(_cfg(), "muon")
        losses = [_step(m, eng, opt, mine(s)) for s in range(10)]
        path = os.path.join(tmp, "iter-000010-ckpt.pth")
        state = {"model": eng.full_state_dict(), "optimizer": opt.state_dict(), "iter_num": 10, "step_count": 10}
        ckpt.save_anywhere(path, state, rank=rank)
        loss11 = _step(m, eng, opt, mine(10))
        # fresh objects, different init, restored from the file
        torch.manual_seed(123)
        m2, eng2, opt2 = _build(_cfg(), "muon")
        with torch.no_grad():
            for g in eng2.groups():
                g.master.add_(1.0)
        st = ckpt.load_anywhere(path)
        eng2.load_full_state_dict(st["model"])
        opt2.load_state_dict(st["optimizer"])
        loss11b = _step(m2, eng2, opt2, mine(10))
        ok_bitwise = bool(torch.equal(loss11, loss11b))
        if rank == 0:
            q.put({"losses": [float(l) for l in losses], "loss11": float(loss11), "loss11b": float(loss11b),
                   "bitwise": ok_bitwise, "keys": sorted(st["model"].keys())[:4], "n_keys": len(st["model"])})
        else:
            assert ok_bitwise
    finally:
        _leave_together()


def test_config1_two_ranks_ten_steps_save_reload_bitwise():
    ctx = mp.get_context("spawn")
    q = ctx.SimpleQueue()
    with tempfile.TemporaryDirectory() as tmp:
        mp.spawn(_worker, args=(2, 29611, tmp, q), nprocs=2, join=True)
    r = q.get()
    assert r["bitwise"], (r["loss11"], r["loss11b"])
    assert r["losses"][-1] < r["losses"][0]
    assert r["n_keys"] == 2 * 8 + 3          # 8 tensors per block + wte, ln_f, lm_head
    assert r["keys"][0] == "lm_head.weight"


def _worker_equiv(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        data = _data(1, 3, per_rank=4)          # the same global batch of 4 rows as the single-process run
        m, eng, opt = _build(_cfg(mup=True, depth_scale=True, use_muon=True, use_muonh=True, head_init_std=0.02), "muonh")
        losses = []
        for s in range(3):
            l = _step(m, eng, opt, data[s, rank * 2:(rank + 1) * 2])
            dist.all_reduce(l)
            losses.append(float(l) / world)
        if rank == 0:
            q.put(losses)
    finally:
        _leave_together()


def test_two_ranks_match_single_process_muonh():
    """Sharded MuonH on 2 ranks follows the single-process trajectory on the same global batch."""
    data = _data(1, 3, per_rank=4)
    m, eng, opt = _build(_cfg(mup=True, depth_scale=True, use_muon=True, use_muonh=True, head_init_std=0.02), "muonh")
    single = [float(_step(m, eng, opt, data[s])) for s in range(3)]
    ctx = mp.get_context("spawn")
    q = ctx.SimpleQueue()
    mp.spawn(_worker_equiv, args=(2, 29612, q), nprocs=2, join=True)
    multi = q.get()
    for a, b in zip(single, multi):
        assert abs(a - b) < 2e-3, (single, multi)


def test_engine_state_dict_names_and_roundtrip():
    m, eng, opt = _build(_cfg(qk_norm=True), "adamw")
    sd = eng.full_state_dict()
    assert {"lm_head.weight", "transformer.wte.weight", "transformer.ln_f.weight", "transformer.h.0.norm_1.weight",
            "transformer.h.0.attn.q_proj.weight", "transformer.h.0.attn.q_norm.weight",
            "transformer.h.1.mlp.w1.weight", "transformer.h.1.mlp.w3.weight"} <= set(sd)
    assert sd["transformer.h.0.mlp.w1.weight"].shape == (2048, 256)
    ref = GPT(_cfg(qk_norm=True))
    ref.load_state_dict(sd)                      # a plain model loads the consolidated checkpoint
    idx = torch.randint(0, 32000, (1, 64))
    ref.compute_dtype = torch.float32
    assert torch.allclose(ref(idx).logits, m(idx).logits, atol=1e-5)


def test_tied_embeddings_and_grad_accumulation():
    cfg = _cfg(tied_embed=True, vocab_size=512)
    m, eng, opt = _build(cfg, "adamw")
    assert m.lm_head.weight is m.transformer.wte.weight
    data = torch.randint(0, 512, (4, 65))
    for mb in (data[:2], data[2:]):
        out = m(mb[:, :-1], use_flce_loss=True)
        eng.backward(fused_linear_cross_entropy(out.logits, out.weight, mb[:, 1:]) / 2)
    g_accum = torch.cat([g.grad.clone() for g in eng.groups()])
    opt.zero_grad()
    out = m(data[:, :-1], use_flce_loss=True)
    eng.backward(fused_linear_cross_entropy(out.logits, out.weight, data[:, 1:]))
    g_full = torch.cat([g.grad.clone() for g in eng.groups()])
    assert torch.allclose(g_accum, g_full, atol=1e-5)


def test_latest_checkpoint_skips_truncated_file(tmp_path):
    good = tmp_path / "iter-000010-ckpt.pth"
    bad = tmp_path / "iter-000020-ckpt.pth"
    torch.save({"iter_num": 10}, good)
    torch.save({"iter_num": 20}, bad)
    raw = bad.read_bytes()
    bad.write_bytes(raw[: len(raw) // 2])
    assert ckpt.latest_ckpt_in_dir(str(tmp_path)) == str(good)
    assert ckpt.find_resume_path("auto", str(tmp_path)) == str(good)
    assert ckpt.find_resume_path(False, str(tmp_path)) is None


def _worker_hsdp(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        mesh = build_mesh(dp=2)
        assert (mesh.dp, mesh.fsdp) == (2, 2) and mesh.data_world == 4
        data = _data(1, 3, per_rank=4, T=64)     # one global batch of 4 rows, one row per rank
        torch.manual_seed(0)
        m = GPT(_cfg(block_size=64, vocab_size=512))
        m.reset_parameters()
        m.compute_dtype = torch.float32
        eng = FSDPEngine(m, mesh, unit_classes=(Block,), param_dtype=torch.float32)
        opt = ShardedOptimizer(eng, lr=1e-3, betas=(0.9, 0.95), algorithm="muonh", mu=0.95, nesterov=True, weight_decay=0.0)
        # shards are 1/2 of each unit (sharded inside a replica), not 1/4
        g0 = next(iter(eng.groups()))
        assert g0.world == 2 and g0.shard_numel * 2 == g0.padded
        losses = []
        for s in range(3):
            l = _step(m, eng, opt, data[s, rank:rank + 1] % 512)
            dist.all_reduce(l)
            losses.append(float(l) / world)
        # the two replicas hold identical shards after training
        mine = torch.cat([g.master for g in eng.groups()])
        other = [torch.empty_like(mine) for _ in range(2)]
        dist.all_gather(other, mine, group=mesh.dp_group)
        same = bool(torch.equal(other[0], other[1]))
        if rank == 0:
            q.put((losses, same))
        else:
            assert same
    finally:
        _leave_together()


def test_hybrid_sharding_dp2_fsdp2_matches_single_process():
    """dp_replicate = 2: gradients are reduce-scattered inside a replica and all-reduced across replicas."""
    data = _data(1, 3, per_rank=4, T=64) % 512
    torch.manual_seed(0)
    m = GPT(_cfg(block_size=64, vocab_size=512))
    m.reset_parameters()
    m.compute_dtype = torch.float32
    eng = FSDPEngine(m, build_mesh(), unit_classes=(Block,), param_dtype=torch.float32)
    opt = ShardedOptimizer(eng, lr=1e-3, betas=(0.9, 0.95), algorithm="muonh", mu=0.95, nesterov=True, weight_decay=0.0)
    single = [float(_step(m, eng, opt, data[s])) for s in range(3)]
    ctx = mp.get_context("spawn")
    q = ctx.SimpleQueue()
    mp.spawn(_worker_hsdp, args=(4, 29613, q), nprocs=4, join=True)
    multi, same = q.get()
    assert same
    for a, b in zip(single, multi):
        assert abs(a - b) < 2e-3, (single, multi)
