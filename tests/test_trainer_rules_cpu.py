"""Trainer rules that only show up over many iterations: per-iteration optimizer hyper-parameters (independent weight
decay, batch ramp-up, beta schedule), the hadam optimizer pair, host offload of master / optimizer shards, a validation
loader that can be read again, and device-status / abort propagation."""
import math

import pytest
import torch

from archscale_b200 import Config
from archscale_b200.data.packed_dataset import PinnedBatchLoader
from archscale_b200.models.gpt import GPT, Block
from archscale_b200.ops import fused_linear_cross_entropy
from archscale_b200.optim import scalar_opts
from archscale_b200.optim.sharded import ShardedOptimizer
from archscale_b200.parallel.fsdp import FSDPEngine
from archscale_b200.train.pretrain import BaseHyperparameters, apply_batch_size_scaling, step_hparams


def test_v2scale_independent_weight_decay():
    # reference: param_group["weight_decay"] = weight_decay / learning_rate / lr_mult, then torch applies lr_group·wd_group
    lr, peak, wd, mult = 3e-4, 4e-4, 0.1, 0.5
    hp = step_hparams("scaling_mup_v2scale", lr=lr, learning_rate=peak, weight_decay=wd, vector_decay=0.0,
                      matrix_lr_mult=mult, super_mup=False)
    assert hp["vector"]["weight_decay"] is None                       # vectors have no decay: untouched
    assert hp["matrix"]["weight_decay"] == pytest.approx(wd / peak / mult)
    # effective decay factor of the weight class per step = lr/peak · wd, independent of the LR multiplier
    assert (lr * mult) * hp["matrix"]["weight_decay"] == pytest.approx(wd * lr / peak)
    plain = step_hparams("scaling_mup", lr=lr, learning_rate=peak, weight_decay=wd, vector_decay=0.0, matrix_lr_mult=mult,
                         super_mup=False)
    assert plain["matrix"] == {"lr_mult": mult, "weight_decay": None, "betas": None, "eps": None}


def test_super_mup_beta_schedule_only_on_decayed_groups():
    hp = step_hparams("scaling_super_mup", lr=2e-4, learning_rate=4e-4, weight_decay=0.1, vector_decay=0.0,
                      matrix_lr_mult=1.0, super_mup=True)
    assert hp["matrix"]["betas"] == pytest.approx((0.95 - 0.10 * 0.5, 0.975 - 0.05 * 0.5))
    assert hp["vector"]["betas"] is None


def test_ramp_iteration_uses_batch_scaled_values():
    hps = BaseHyperparameters()
    sc = apply_batch_size_scaling(0.25, hps, "sdew")
    hp = step_hparams("scaling_mup_v2scale", lr=1e-4, learning_rate=sc["learning_rate"], weight_decay=0.1,
                      vector_decay=0.0, matrix_lr_mult=0.5, super_mup=False, ramp=sc)
    assert hp["matrix"]["eps"] == sc["eps"] == hps.eps / 0.5
    assert hp["matrix"]["betas"] == (sc["beta1"], sc["beta2"]) and hp["vector"]["betas"] == (sc["beta1"], sc["beta2"])
    assert hp["matrix"]["weight_decay"] == pytest.approx(sc["weight_decay"] / sc["learning_rate"] / 0.5)
    assert hp["vector"]["weight_decay"] is None
    # the reference's default rule scales the peak LR with the square root of the batch ratio
    assert apply_batch_size_scaling(4.0, hps, "default")["learning_rate"] == pytest.approx(hps.eta0 * 2)


def test_nadam_rule_matches_torch():
    torch.manual_seed(0)
    w = torch.randn(8, 5)
    ref = torch.nn.Parameter(w.clone())
    opt = torch.optim.NAdam([ref], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, decoupled_weight_decay=True)
    x, m, v = w.clone(), torch.zeros_like(w), torch.zeros_like(w)
    prod = 1.0
    for step in range(1, 6):
        g = torch.randn(8, 5)
        ref.grad = g.clone()
        opt.step()
        prod = scalar_opts.nadam_update_foreach([x], [g], [m], [v], 1e-2, 0.9, 0.95, 0.1, step, 1e-8, prod)
        assert torch.allclose(x, ref.detach(), atol=1e-6), step


def _cfg():
    return Config.from_name("transformer_gqa4_d8", n_layer=2, ar=None, n_embd=64, n_head=2, n_query_groups=1, head_dim=32,
                            intermediate_size=128, vocab_size=256, padding_multiple=64, block_size=32, mup=True)


def _build(algorithm, **kw):
    torch.manual_seed(0)
    m = GPT(_cfg())
    m.reset_parameters()
    m.compute_dtype = torch.float32
    eng = FSDPEngine(m, unit_classes=(Block,), param_dtype=torch.float32)
    opt = ShardedOptimizer(eng, lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, weight_lr_mult=0.5,
                           algorithm=algorithm, **kw)
    return m, eng, opt


def _step(m, eng, opt, batch, **kw):
    out = m(batch[:, :-1], use_flce_loss=True)
    loss = fused_linear_cross_entropy(out.logits, out.weight, batch[:, 1:])
    eng.backward(loss)
    opt.step(**kw)
    opt.zero_grad()
    return float(loss)


def test_hadam_is_adamw_for_vectors_and_nadam_for_weights():
    data = torch.randint(0, 256, (3, 2, 33), generator=torch.Generator().manual_seed(0))
    m, eng, opt = _build("hadam", vector_betas=(0.8, 0.95), vector_eps=1e-10)
    # the same model under two torch optimizers, grouped by the reference's name rule
    torch.manual_seed(0)
    ref = GPT(_cfg())
    ref.reset_parameters()
    ref.compute_dtype = torch.float32
    from archscale_b200.utils.param_groups import is_vector_param
    vec = [p for n, p in ref.named_parameters() if is_vector_param(n)]
    mat = [p for n, p in ref.named_parameters() if not is_vector_param(n)]
    o1 = torch.optim.AdamW(vec, lr=1e-2, betas=(0.8, 0.95), eps=1e-10, weight_decay=0.0)
    o2 = torch.optim.NAdam(mat, lr=1e-2 * 0.5, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, decoupled_weight_decay=True)
    for s in range(3):
        _step(m, eng, opt, data[s])
        out = ref(data[s][:, :-1], use_flce_loss=True)
        fused_linear_cross_entropy(out.logits, out.weight, data[s][:, 1:]).backward()
        o1.step(); o2.step(); o1.zero_grad(); o2.zero_grad()
        sd = eng.full_state_dict()
        # the first step is exact; afterwards rounding differences of near-zero gradient entries are amplified by the
        # division by sqrt(v), so later steps are compared at the size of one update (lr = 5e-3 .. 1e-2)
        tol = 1e-6 if s == 0 else 2e-3
        for n, p in ref.named_parameters():
            assert torch.allclose(sd[n], p.detach(), atol=tol), (s, n, float((sd[n] - p.detach()).abs().max()))


def test_cpu_offload_changes_nothing_but_where_the_shards_wait():
    data = torch.randint(0, 256, (3, 2, 33), generator=torch.Generator().manual_seed(0))
    m, eng, opt = _build("muonh")
    plain = [_step(m, eng, opt, data[s]) for s in range(3)]
    ref_sd = eng.full_state_dict()
    m, eng, opt = _build("muonh")
    eng.enable_cpu_offload([opt.m, opt.v])
    eng.offload_states()
    off = []
    for s in range(3):
        assert all(g.master is None for g in eng.groups() if g.dtype != torch.float32)      # shards wait on the host
        assert all(opt.m[id(g)] is None for g in eng.groups() if g.dtype != torch.float32)
        off.append(_step(m, eng, opt, data[s]))
        eng.offload_states()
    assert plain == off
    sd = eng.full_state_dict()                      # reloads by itself
    assert all(torch.equal(sd[k], ref_sd[k]) for k in ref_sd)


def test_exhausted_loader_keeps_raising_and_fresh_loader_repeats_batches():
    def stream():
        return iter([torch.full((4,), i) for i in range(5)])
    a = PinnedBatchLoader(stream(), 2, pin=False)
    got = [b for b, _ in a]
    assert len(got) == 2                           # 5 samples → two full batches
    with pytest.raises(StopIteration):
        next(a)                                    # must not block once the stream has ended
    b = PinnedBatchLoader(stream(), 2, pin=False)
    assert torch.equal(next(b)[0], got[0])         # a fresh loader yields the same leading batches
    b.close()


def test_raised_exception_reaches_the_peers_check():
    import torch.distributed as dist
    from archscale_b200.utils.health import Heartbeat, PeerFailure
    store = dist.HashStore()
    h0, h1 = Heartbeat(store, 0, 2), Heartbeat(store, 1, 2)
    h1.check()
    with pytest.raises(ZeroDivisionError):
        with h0.guard():
            1 / 0
    with pytest.raises(PeerFailure, match="rank 0 reported a failure"):
        h1.check()


@pytest.mark.parametrize("reduction", ["mean", "sum", "none"])
def test_fused_cross_entropy_module_matches_oracle(reduction):
    from archscale_b200.ops import FusedCrossEntropyLoss, cross_entropy_ref
    torch.manual_seed(0)
    logits = torch.randn(12, 50, requires_grad=True)
    tgt = torch.randint(0, 50, (12,))
    tgt[3] = -100
    mod = FusedCrossEntropyLoss(label_smoothing=0.1, lse_square_scale=1e-3, reduction=reduction)
    a = mod(logits, tgt)
    ref_in = logits.detach().clone().requires_grad_()
    b = cross_entropy_ref(ref_in, tgt, -100, 0.1, 1e-3, reduction)
    assert torch.allclose(a, b, atol=1e-5)
    w = torch.randn_like(a)
    (a * w).sum().backward()
    (b * w).sum().backward()
    assert torch.allclose(logits.grad, ref_in.grad, atol=1e-5)


def test_fp4_flag_selects_nvfp4_linears_and_not_mxfp8():
    from archscale_b200.train.pretrain import make_plan
    kw = dict(train_model="transformer_gqa4", train_name="scaling_mup_muonh", depth=8, max_tokens=1e6, ctx_len=64, swa_len=None,
              data_mixture=None, fsdp_save_mem=False, save_step=None, base_hps=BaseHyperparameters(), micro_bsz=1,
              total_bsz=64, yarn_scale=1.0, sparsity=1, top_k=2, use_flce=True, norm_class=None, fp8=False, post_norm=None,
              bramp_ratio=None, aux_style=None, aux_gamma=None, num_extrp=None, offloading=False, act_ckpt=False,
              share_expert=None, global_aux=None, sqrt_gate=None, head_init_std=0.02, ar=None, load_dir=None, world_size=1,
              local_world_size=1)
    plan4 = make_plan(fp4=True, **kw)
    assert plan4.overrides.get("nvfp4") and not plan4.overrides.get("mxfp8")
    plan8 = make_plan(fp4=False, **{**kw, "fp8": True})
    assert plan8.overrides.get("mxfp8") and not plan8.overrides.get("nvfp4")
    plan = make_plan(fp4=False, **{**kw, "fsdp_save_mem": True})
    assert plan.cpu_offload and plan.activation_checkpointing      # --fsdp_save_mem switches both on


def test_logging_worker_process():
    from archscale_b200.utils import logging_utils as lu
    lu.configure_logging_executor(use_multiprocessing=True)
    try:
        payload = lu.build_logging_payload(10, 5, 1.5, 1.0, optimizer_stats={"betas": (0.9, 0.95), "eps": 1e-8, "weight_lr": 1e-3,
                                                                            "vector_lr": 1e-3, "weight_decay": 0.0})
        lu.submit_logging_task(payload)
        got = {}
        lu.wait_for_logging_tasks(lambda d, step: got.update(d, step=step), lambda s: None)
        assert got["step"] == 5 and any(k.startswith("metric/") or k.startswith("optim") or "grad" in k for k in got)
    finally:
        lu.shutdown()


def test_deferred_clip_equals_clip_in_place():
    data = torch.randint(0, 256, (2, 2, 33), generator=torch.Generator().manual_seed(0))

    def run(defer):
        m, eng, opt = _build("muonh")
        for s in range(2):
            out = m(data[s][:, :-1], use_flce_loss=True)
            eng.backward(fused_linear_cross_entropy(out.logits, out.weight, data[s][:, 1:]) * 50.0)   # large gradients: clip bites
            if defer:
                gn, coef = eng.clip_grad_norm_(1.0, defer=True)
                assert float(coef) < 1.0
                opt.step(grad_scale=coef)
            else:
                gn = eng.clip_grad_norm_(1.0)
                opt.step()
            opt.zero_grad()
        return eng.full_state_dict(), float(gn)

    a, ga = run(False)
    b, gb = run(True)
    assert ga == gb
    assert all(torch.allclose(a[k], b[k], atol=1e-6) for k in a)


def test_residual_stream_dtype_follows_the_flag():
    """``residual_in_fp32`` decides the type of the residual stream between the blocks (fp32, or the compute dtype)."""
    from archscale_b200 import Config
    from archscale_b200.models.gpt import GPT
    seen = {}

    def run(flag):
        torch.manual_seed(0)
        cfg = Config.from_name("transformer_gqa4_d8", n_layer=2, ar=None, n_embd=64, n_head=2, n_query_groups=1, head_dim=32,
                               intermediate_size=128, vocab_size=128, padding_multiple=64, block_size=32, residual_in_fp32=flag)
        model = GPT(cfg).bfloat16()
        model.reset_parameters()
        model.compute_dtype = torch.bfloat16
        dtypes = []
        h = model.transformer.h[1].norm_1.register_forward_pre_hook(lambda m, args: dtypes.append(args[0].dtype))
        out = model(torch.randint(0, 128, (2, 16)))
        h.remove()
        seen[flag] = (dtypes[0], out.logits.float())

    run(True)
    run(False)
    assert seen[True][0] == torch.float32 and seen[False][0] == torch.bfloat16
    a, b = seen[True][1], seen[False][1]
    assert torch.isfinite(a).all() and torch.isfinite(b).all()
    assert float((a - b).norm() / a.norm()) < 0.1          # same model, the stream's rounding is the only difference
