"""Checkpoints written under tensor / expert parallelism hold whole tensors: they load into an unsplit model, and a
resumed parallel run continues on the same trajectory (two gloo ranks, fp32)."""
import os

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


def _dense_cfg():
    return Config.from_name("transformer_gqa4_d8", n_layer=2, ar=None, n_embd=128, n_head=4, n_query_groups=2, head_dim=32,
                            intermediate_size=256, vocab_size=512, padding_multiple=64, block_size=64, qk_norm=True)


def _moe_cfg(ep):
    return Config.from_name("transformer_gqa4_h2_moe_s2_k2_d8", n_layer=2, ar=None, n_embd=64, n_head=2, n_query_groups=1,
                            head_dim=32, intermediate_size=128, vocab_size=512, padding_multiple=64, block_size=32,
                            ep_size=ep)


def _build(cfg, mesh, parallel):
    torch.manual_seed(0)
    m = GPT(cfg)
    m.reset_parameters()
    m.compute_dtype = torch.float32
    if parallel == "tp" and mesh.tp > 1:
        tp_mod.apply_tensor_parallel(m, mesh)
    if parallel == "ep" and mesh.ep > 1:
        from archscale_b200.parallel import ep as ep_mod
        ep_mod.attach(m, mesh)
    eng = FSDPEngine(m, mesh, unit_classes=(Block,), param_dtype=torch.float32)
    opt = ShardedOptimizer(eng, lr=1e-2, betas=(0.9, 0.95), algorithm="adamw", weight_decay=0.0)
    return m, eng, opt


def _step(m, eng, opt, mesh, batch, update=True):
    out = m(batch[:, :-1], use_flce_loss=True)
    tgt = batch[:, 1:]
    if mesh.tp > 1:
        tgt = tp_mod.token_slice(tgt, mesh.tp, mesh.tp_rank).contiguous()
    loss = fused_linear_cross_entropy(out.logits, out.weight, tgt)
    if not update:
        return loss.detach()
    back = loss / mesh.tp
    if m.config.moe:
        back = back + m.aux_loss
    eng.backward(back)
    tp_mod.sync_replicated_grads(eng, mesh)
    eng.clip_grad_norm_(1.0)
    opt.step()
    opt.zero_grad()
    return loss.detach()


def _worker(rank, world, port, q, parallel, tmp):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        mesh = build_mesh(dp=1, tp=2) if parallel == "tp" else build_mesh(dp=1, tp=1, ep=2)
        cfg = _dense_cfg() if parallel == "tp" else _moe_cfg(2)
        T = cfg.block_size
        data = torch.randint(0, 512, (4, 2, T + 1), generator=torch.Generator().manual_seed(0 if parallel == "tp" else rank))
        m, eng, opt = _build(cfg, mesh, parallel)
        for s in range(2):
            _step(m, eng, opt, mesh, data[s])
        sd, osd = eng.full_state_dict(rank0_only=False), opt.state_dict(rank0_only=False)
        at_save = float(_step(m, eng, opt, mesh, data[3], update=False))
        cont = float(_step(m, eng, opt, mesh, data[2]))
        cont2 = float(_step(m, eng, opt, mesh, data[3], update=False))
        # resume: a fresh parallel model loads the whole-tensor checkpoint and repeats step 3
        m2, eng2, opt2 = _build(cfg, mesh, parallel)
        eng2.load_full_state_dict(sd)
        opt2.load_state_dict(osd)
        res = float(_step(m2, eng2, opt2, mesh, data[2]))
        res2 = float(_step(m2, eng2, opt2, mesh, data[3], update=False))
        if rank == 0:
            # tensors go through a file: a queue would hand over shared-memory handles of a process that is about to exit
            torch.save({"sd": sd, "osd": osd, "eval_batch": data[3]}, os.path.join(tmp, "out.pt"))
            q.put({"cont": (cont, cont2), "res": (res, res2), "at_save": at_save})
    finally:
        _leave_together()


def _spawn(parallel):
    import tempfile
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    with tempfile.TemporaryDirectory() as tmp:
        procs = [ctx.Process(target=_worker, args=(r, 2, port, q, parallel, tmp)) for r in range(2)]
        for p in procs:
            p.start()
        out = q.get(timeout=300)
        for p in procs:
            p.join(timeout=120)
            assert p.exitcode == 0
        out.update(torch.load(os.path.join(tmp, "out.pt")))
    return out


def test_tp2_checkpoint_is_whole_and_resumes():
    r = _spawn("tp")
    sd, osd = r["sd"], r["osd"]
    assert sd["transformer.h.0.attn.q_proj.weight"].shape == (128, 128)
    assert sd["transformer.h.0.mlp.w1.weight"].shape == (512, 128) and sd["transformer.h.0.mlp.w3.weight"].shape == (128, 256)
    assert osd["state"]["transformer.h.1.mlp.w3.weight"]["momentum"].shape == (128, 256)
    assert r["cont"] == r["res"], (r["cont"], r["res"])          # resumed run: identical losses
    # the unsplit single-process model reaches the same weights on the same data and loads the checkpoint as is
    mesh1 = Mesh(world=1, rank=0, dp=1, fsdp=1, tp=1)
    data = torch.randint(0, 512, (4, 2, 65), generator=torch.Generator().manual_seed(0))
    m, eng, opt = _build(_dense_cfg(), mesh1, "none")
    for s in range(2):
        _step(m, eng, opt, mesh1, data[s])
    ref = eng.full_state_dict()
    for k in ref:
        assert sd[k].shape == ref[k].shape, k
        assert torch.allclose(sd[k], ref[k], atol=2e-4), (k, float((sd[k] - ref[k]).abs().max()))
    plain = GPT(_dense_cfg())
    plain.load_state_dict(sd)


def test_ep2_checkpoint_is_whole_and_resumes():
    r = _spawn("ep")
    sd, osd = r["sd"], r["osd"]
    cfg1 = _moe_cfg(1)
    E = cfg1.routed_experts
    assert sd["transformer.h.0.mlp.mods_in.weight"].shape[0] == E
    assert osd["state"]["transformer.h.0.mlp.mods_in.weight"]["momentum"].shape[0] == E
    assert osd["state"]["transformer.h.0.mlp.mods_in.weight"]["variance"].shape[0] == E
    # the two ranks own different experts: the second half of the momentum is not a copy of the first
    mom = osd["state"]["transformer.h.0.mlp.mods_in.weight"]["momentum"]
    assert not torch.equal(mom[:E // 2], mom[E // 2:])
    assert r["cont"] == r["res"], (r["cont"], r["res"])
    # a single-process model with all experts loads the checkpoint and computes rank 0's evaluation loss
    plain = GPT(cfg1)
    plain.load_state_dict(sd)
    plain.compute_dtype = torch.float32
    b = r["eval_batch"]
    out = plain(b[:, :-1], use_flce_loss=True)
    loss = float(fused_linear_cross_entropy(out.logits, out.weight, b[:, 1:]))
    assert abs(loss - r["at_save"]) < 2e-4, (loss, r["at_save"])


def test_localize_rejects_wrong_size():
    mesh1 = Mesh(world=1, rank=0, dp=1, fsdp=1, tp=1)
    m, eng, opt = _build(_dense_cfg(), mesh1, "none")
    sd = eng.full_state_dict()
    sd["transformer.h.0.mlp.w3.weight"] = sd["transformer.h.0.mlp.w3.weight"][:, :100]
    try:
        eng.load_full_state_dict(sd)
    except ValueError as e:
        assert "expected" in str(e)
    else:
        raise AssertionError("a truncated tensor loaded silently")
