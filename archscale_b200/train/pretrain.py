"""Pre-training entry point: flags, hyper-parameter laws, train / validate loops, resume.

Public surface of the reference trainer (`pretrain.py:172-216` flags of ``setup()``,
`:266-271,466-496` train-name switches, `:305-378` token / batch / LR / WD laws, `:565-592`
parameter groups, `:728-1020` train loop, `:1022-1086` validate, `:1280-1309` LR schedule,
`:1313-1323` resume) without Lightning Fabric / jsonargparse: one process per GPU under
``torchrun`` (or a single process), :class:`archscale_b200.parallel.fsdp.FSDPEngine` for
sharding and :class:`archscale_b200.optim.sharded.ShardedOptimizer` for the update.

Run:  ``torchrun --nproc-per-node 8 pretrain.py --train_data_dir DIR --train_model transformer_gqa4
--depth 16 --train_name scaling_mup_muonh_qknorm --fsdp2 true --micro_bsz 8``.
``--train_data_dir synthetic`` trains on uniform-random tokens (benchmarks, smoke tests).

Differences from the reference that matter to users: the loss value is only copied to the host
on logging steps (the reference synchronises every micro-step, `pretrain.py:1009`);
``--micro_bsz`` is honoured for every context length unless ``_varlen`` packs one row;
resume seeks the data stream in O(1) instead of replaying batches.
"""
from __future__ import annotations

import contextlib
import dataclasses
import glob
import json
import math
import os
import random
import re
import sys
import time
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple, Union

import torch

from archscale_b200.config import Config, get_parameters_count
from archscale_b200.data.packed_dataset import CombinedDataset, PackedDataset, PinnedBatchLoader, SyntheticTokens
from archscale_b200.models.gpt import GPT, Block
from archscale_b200.ops.cross_entropy import FusedCrossEntropyLoss, FusedLinearCrossEntropyLoss
from archscale_b200.optim.sharded import VECTOR_NAMES, ShardedOptimizer
from archscale_b200.parallel import dist_utils as du
from archscale_b200.parallel.fsdp import FSDPEngine
from archscale_b200.parallel.mesh import Mesh, build_mesh
from archscale_b200.utils import checkpoint as ckpt
from archscale_b200.utils import init as init_utils
from archscale_b200.utils import logging_utils as lu
from archscale_b200.utils.misc import num_parameters
from archscale_b200.utils.speed_monitor import (DeviceStepTimer, SpeedMonitor, estimate_flops, get_flops_available,
                                                 matmul_parameter_count)

RNG_SEED = 3407


@dataclass
class BaseHyperparameters:
    """Base point of the μP++ / HyperP transfer rules (`pretrain.py:82-99`)."""
    d0: int = 8
    eta0: float = 6e-4
    b0: int = 2 ** 21
    t0: Union[int, float] = int(9.5e9)
    hd0: int = 128
    w_init_scale: float = 1.0
    n0_mult: float = 237568
    weight_decay: float = 1e-1
    eps: float = 1e-8
    min_lr_mult: float = 0.0
    warmup_tokens: Union[int, float] = int(1e9)
    beta1: float = 0.9
    beta2: float = 0.95
    muon_beta: float = 0.95
    weight_lr_scale: float = 1


def apply_batch_size_scaling(batch_ratio: float, hps: BaseHyperparameters, mode: Optional[str] = "sdew") -> Dict[str, float]:
    """Batch-size transfer rules: "sde" (Adam), "sdew" (AdamW), "default" (√ LR), None (constant)."""
    out = dict(learning_rate=hps.eta0, eps=hps.eps, beta1=hps.beta1, beta2=hps.beta2, weight_decay=hps.weight_decay)
    r = math.sqrt(batch_ratio)
    if mode == "sde":
        out.update(learning_rate=hps.eta0 * r, eps=hps.eps / r, beta2=1 - (1 - hps.beta2) * batch_ratio)
    elif mode == "sdew":
        out.update(eps=hps.eps / r, beta2=1 - (1 - hps.beta2) * r, weight_decay=hps.weight_decay * r)
    elif mode == "default":
        out.update(learning_rate=hps.eta0 * r)
    return out


def batch_size_rampup_func(iters: int, max_iters: int, batch_size_ratio: float = 4.0) -> float:
    ramp = max(int(0.05 * max_iters), 1)
    if iters >= ramp:
        return batch_size_ratio
    return 1.0 + (batch_size_ratio - 1.0) * iters / ramp


def get_lr(it: int, warmup_iters: int, max_iters: int, lr: float, min_lr_mult: float = 0.0, train_name: str = "") -> float:
    """Linear warm-up → optional WSD plateau (5/7 of the rest) → linear or cosine decay."""
    if it < warmup_iters:
        return lr * it / warmup_iters
    if it > max_iters:
        return min_lr_mult * lr
    if "wsd" in train_name:
        stable = int(5 / 7 * (max_iters - warmup_iters))
        if it < warmup_iters + stable:
            return lr
        ratio = (it - warmup_iters - stable) / (max_iters - warmup_iters - stable)
    else:
        ratio = (it - warmup_iters) / (max_iters - warmup_iters)
    if "cosine" in train_name:
        return min_lr_mult * lr + 0.5 * (1.0 + math.cos(math.pi * ratio)) * (lr - min_lr_mult * lr)
    return lr + ratio * (min_lr_mult * lr - lr)


def step_hparams(train_config: str, *, lr: float, learning_rate: float, weight_decay: float, vector_decay: float,
                 matrix_lr_mult: float, super_mup: bool, ramp: Optional[Dict[str, float]] = None) -> Dict[str, Dict[str, Any]]:
    """Optimizer hyper-parameters of one iteration for the two parameter classes, as the reference's ``update_param``
    sets them on its param groups every iteration (`pretrain.py:829-878`).

    ``lr`` is the scheduled value, ``learning_rate`` the peak it decays from, ``matrix_lr_mult`` the weight group's
    LR multiplier (``d0/depth`` for AdamW-family runs, × ``weight_lr_scale`` for the hybrid ones).  ``ramp`` holds the
    batch-size-scaled values on the iterations where the batch ramp-up changes the accumulation count.  A value of
    ``None`` means "leave what the optimizer has".  Rules, per class with its own ``wd`` and ``lr_mult``:

    * ramp iteration: ``eps``, ``betas`` ← scaled values; if ``wd > 0``: ``wd`` ← scaled weight decay, and for
      ``v2scale`` runs divided by ``learning_rate·lr_mult`` (independent weight decay: the decay per step is
      ``wd·lr/learning_rate`` whatever the LR multipliers);
    * otherwise, if ``wd > 0``: ``v2scale`` → ``wd = weight_decay/(learning_rate·lr_mult)``; ``super_mup`` → betas follow
      the LR schedule, ``(0.95 − 0.10·lr/learning_rate, 0.975 − 0.05·lr/learning_rate)``.
    """
    out: Dict[str, Dict[str, Any]] = {}
    v2 = "v2scale" in train_config
    frac = lr / learning_rate if learning_rate else 0.0
    for cls, wd, mult in (("vector", vector_decay, 1.0), ("matrix", weight_decay, matrix_lr_mult)):
        h: Dict[str, Any] = {"lr_mult": mult, "weight_decay": None, "betas": None, "eps": None}
        if ramp is not None:
            h["eps"], h["betas"] = ramp["eps"], (ramp["beta1"], ramp["beta2"])
            if wd > 0:
                h["weight_decay"] = ramp["weight_decay"] / learning_rate / mult if v2 else ramp["weight_decay"]
        elif wd > 0:
            if v2:
                h["weight_decay"] = weight_decay / learning_rate / mult
            if super_mup:
                h["betas"] = (0.95 - (0.95 - 0.85) * frac, 0.975 - (0.975 - 0.925) * frac)
        out[cls] = h
    return out


@dataclass
class TrainPlan:
    """Everything ``setup()`` derives from the flags before any tensor is created."""
    model_name: str = ""
    base_model_name: str = ""
    train_config: str = ""
    name: str = ""
    out_dir: str = ""
    seq_len: int = 4096
    micro_batch_size: int = 2
    global_batch_size: int = 0
    batch_size: int = 0
    gradient_accumulation_steps: int = 1
    train_tokens: int = 0
    learning_rate: float = 0.0
    weight_decay: float = 0.0
    eps: float = 1e-8
    beta1: float = 0.9
    beta2: float = 0.95
    muon_beta: float = 0.95
    weight_lr_scale: float = 1.0
    warmup_tokens: int = 0
    min_lr: float = 0.0
    mup: bool = False
    original_mup: bool = False
    super_mup: bool = False
    depth: int = 16
    label_smoothing: float = 0.0
    use_flce_loss: bool = False
    use_cu_seqlen: bool = False
    grad_clip: float = 1.0
    log_step_interval: int = 10
    save_step_interval: int = 1000
    eval_step_interval: int = 1000
    eval_iters: int = 50
    num_extrapol: int = 4
    data_chunks: int = 8
    bsz_rampup_ratio: int = 1
    bsz_scaling: str = "default"
    cpu_offload: bool = False
    activation_checkpointing: bool = False
    code_dropout: float = 0.0
    nodes: int = 1
    devices: int = 1
    overrides: Dict[str, Any] = field(default_factory=dict)
    train_data_config: List[Tuple[str, float]] = field(default_factory=lambda: [("train", 1.0)])
    val_data_config: List[Tuple[str, float]] = field(default_factory=lambda: [("validation", 1.0)])


def make_plan(*, train_model: Optional[str], train_name: str, depth: int, max_tokens: Optional[float],
              ctx_len: Optional[int], swa_len: Optional[int], data_mixture: Optional[str], fsdp_save_mem: bool,
              save_step: Optional[int], base_hps: BaseHyperparameters, micro_bsz: int, total_bsz: Optional[int],
              yarn_scale: float, sparsity: int, top_k: int, use_flce: Optional[bool], norm_class: Optional[str],
              fp8: bool, fp4: bool, post_norm: Optional[bool], bramp_ratio: Optional[int], aux_style: Optional[str],
              aux_gamma: Optional[float], num_extrp: Optional[int], offloading: bool, act_ckpt: bool,
              share_expert: Optional[bool], global_aux: Optional[bool], sqrt_gate: Optional[bool],
              head_init_std: Optional[float], ar: Optional[int], load_dir: Optional[str], world_size: int,
              local_world_size: int, tp: int = 1, ep: int = 1, extra_overrides: Optional[Dict[str, Any]] = None) -> TrainPlan:
    """Pure function of the flags: names, token budget, batch, LR/WD laws and config overrides."""
    p = TrainPlan()
    hps = base_hps
    p.nodes = max(world_size // max(local_world_size, 1), 1)
    p.devices = max(local_world_size, 1)
    p.seq_len = ctx_len if ctx_len is not None else 4096
    p.num_extrapol = num_extrp if num_extrp is not None else 4
    p.save_step_interval = save_step if save_step is not None else 1000
    model_name = train_model if train_model is not None else "transformer"
    tc = p.train_config = train_name
    p.bsz_rampup_ratio = bramp_ratio if bramp_ratio is not None else 1
    p.data_chunks = 128 if "v2scale" in tc else 8
    if fsdp_save_mem:
        offloading = act_ckpt = True
    # --fp4 selects NVFP4 linears; like the reference (`pretrain.py:250`) it implies the settings --fp8 implies
    low_precision = fp8 or fp4
    if data_mixture is not None:
        with open(data_mixture) as f:
            p.train_data_config = list(json.load(f).items())
    p.depth = depth
    p.mup = "mup" in tc or "muonh" in tc
    p.original_mup = "_ori_mup" in tc
    rope_base = 640_000 if "_rbase_" in tc else 10_000
    p.super_mup = "super_mup" in tc
    p.use_cu_seqlen = "_varlen" in tc
    p.label_smoothing = 0.1 if "_ls_" in tc else 0.0
    if "_moe" in model_name:
        model_name = f"{model_name}_s{sparsity}_k{top_k}"
    p.base_model_name = f"{model_name}_d{hps.d0}"
    p.model_name = model_name = f"{model_name}_d{depth}"
    model_config = Config.from_name(model_name)
    # fixed-size registry entries (e.g. phi4miniflash_d32) have no base-depth sibling; the base is only
    # needed for the token-budget law, i.e. when --max_tokens is not given
    try:
        base_config = Config.from_name(p.base_model_name)
    except KeyError:
        base_config = None
    p.use_flce_loss = use_flce if use_flce is not None else (model_config.vocab_size > 100_000 or "validation" in tc or low_precision)
    name = f"{tc}_{model_name}"
    if ar is not None:
        name += f"_ar{ar}"
    name += f"_ctx{p.seq_len}"
    if swa_len is not None:
        name += f"_swa{swa_len}"
    if p.bsz_rampup_ratio != 1:
        name += f"_bramp{p.bsz_rampup_ratio}"
    p.name = name
    p.out_dir = os.path.join(os.getenv("LIGHTNING_ARTIFACTS_DIR", "out"), name)
    # packed varlen training flattens the batch into one row; otherwise micro_bsz is honoured at any length
    p.micro_batch_size = 1 if p.use_cu_seqlen else micro_bsz
    if max_tokens is not None:
        p.train_tokens = int(max_tokens)
    else:
        if base_config is None:
            raise ValueError(f"{p.base_model_name} is not a registered config: pass --max_tokens for {model_name}")
        if ar is not None:
            model_config.ar = base_config.ar = ar
        n_base = get_parameters_count(p.base_model_name, hps.d0, base_config, tc)
        n_target = get_parameters_count(model_name, depth, model_config, tc)
        p.train_tokens = int(hps.t0 * n_target / n_base)
    raw_b = hps.b0 if total_bsz is None else total_bsz
    data_ranks = max(world_size // tp, 1)
    multiple = data_ranks * p.micro_batch_size * p.seq_len
    b = max(((raw_b + multiple // 2) // multiple) * multiple, multiple)
    hps = dataclasses.replace(hps)
    if "muonball" in tc or "muonh" in tc:
        hps.weight_decay = 0.0
    scaled = apply_batch_size_scaling(b / hps.b0, hps, "default")
    p.learning_rate, p.eps, p.beta1, p.beta2, p.weight_decay = (scaled[k] for k in
                                                               ("learning_rate", "eps", "beta1", "beta2", "weight_decay"))
    depth_mup = p.mup and not p.original_mup
    depth_scale = depth_mup or "_dsca_" in tc
    if depth_mup:
        p.learning_rate *= math.sqrt(hps.d0 / depth)
    if "muonh" in tc:
        p.learning_rate *= (p.train_tokens / hps.t0) ** (-0.32)
    p.min_lr = hps.min_lr_mult
    if "midtrain" in tc or "muon" in tc:
        p.warmup_tokens = 0
    elif p.super_mup:
        p.warmup_tokens = int(hps.warmup_tokens / hps.t0 * p.train_tokens)
    else:
        p.warmup_tokens = int(hps.warmup_tokens)
    p.muon_beta, p.weight_lr_scale = hps.muon_beta, hps.weight_lr_scale
    if "muon" in tc:
        p.weight_decay = p.weight_decay * hps.d0 / depth
    p.global_batch_size = b // (p.seq_len * p.nodes)
    p.batch_size = b // (p.seq_len * data_ranks)
    p.gradient_accumulation_steps = p.batch_size // p.micro_batch_size
    assert p.gradient_accumulation_steps > 0
    total_evals = 400
    p.eval_iters = total_evals // p.micro_batch_size // (2 if p.micro_batch_size == 1 else 1)
    p.cpu_offload, p.activation_checkpointing = offloading, act_ckpt
    # ---- config overrides
    scaling_factor = yarn_scale if ("midtrain" in tc or "validation" in tc) else 1.0
    ov: Dict[str, Any] = {
        "mup": p.mup, "depth_scale": depth_scale, "super_mup": p.super_mup, "mup_d0": hps.d0, "mup_hd0": hps.hd0,
        "w_init_scale": hps.w_init_scale, "block_size": p.seq_len, "use_cu_seqlen": p.use_cu_seqlen,
        "head_init_std": head_init_std, "original_mup": p.original_mup, "rope_base": rope_base, "eos_token_id": 2,
        "scaling_factor": scaling_factor,
    }
    if "validation" in tc and load_dir:
        m = re.search(r"_swa(\d+)", load_dir)
        if m:
            ov["local_window"] = int(m.group(1))
        m = re.search(r"_ctx(\d+)", load_dir)
        if m:
            ov["block_size"] = int(m.group(1))
    for key, val in (("local_window", swa_len), ("ar", ar), ("aux_style", aux_style), ("aux_gamma", aux_gamma),
                     ("_norm_class", norm_class), ("post_norm", post_norm), ("sqrt_gate", sqrt_gate),
                     ("share_expert", share_expert), ("global_aux", global_aux)):
        if val is not None:
            ov[key] = val
    switches = (("_bias", {"attn_bias": True, "attn_out_bias": True, "bias": True}), ("muon", {"use_muon": True}),
                ("muonh", {"use_muonh": True}), ("_tie", {"tied_embed": True}), ("_lc", {"lc": True}),
                ("postnorm_decouple", {"decouple_postnorm": True}), ("_skipgain", {"skip_gain": True}),
                ("_qknorm", {"qk_norm": True}), ("_anorm", {"attn_norm": True}), ("_fnorm", {"ffn_norm": True}),
                ("_nope", {"nope": True}), ("_ga_", {"gated_attn": True}), ("_noskip", {"no_skip": True}),
                ("_noskip_sum", {"sum_skip": True, "no_skip": False}))
    for key, upd in switches:
        if key in tc:
            ov.update(upd)
    if fp4:
        ov["nvfp4"] = True
    elif fp8:
        ov["mxfp8"] = True
    if tp > 1:
        ov["tp_size"] = tp
    if ep > 1:
        ov["ep_size"] = ep
    if extra_overrides:
        ov.update(extra_overrides)
    p.overrides = ov
    return p


# =====================================================================================
class Trainer:
    def __init__(self, plan: TrainPlan, mesh: Mesh, device: torch.device, train_data_dir: str,
                 val_data_dir: Optional[str], resume, load_dir: Optional[str], base_hps: BaseHyperparameters,
                 use_mlflow: bool = False, wandb_project: Optional[str] = None, precision: str = "bf16",
                 fused_comm: bool = False, max_steps: Optional[int] = None, quiet: bool = False,
                 logging_multiprocessing: bool = False) -> None:
        self.plan, self.mesh, self.device, self.base_hps = plan, mesh, device, base_hps
        self.logging_multiprocessing = logging_multiprocessing
        self.rank0 = mesh.rank == 0
        self.quiet = quiet
        self.max_steps = max_steps
        p = plan
        self.config = Config.from_name(p.model_name, **p.overrides)
        torch.manual_seed(RNG_SEED)
        random.seed(RNG_SEED)
        compute_dtype = torch.bfloat16 if precision == "bf16" else torch.float32
        t0 = time.perf_counter()
        with torch.device(device):
            self.model = GPT(self.config)
        self.model.reset_parameters()
        self.model.compute_dtype = compute_dtype
        self.n_params_actual = num_parameters(self.model)
        if self.config.mxfp8:
            from archscale_b200.models.layers import apply_mxfp8
            n_fp8 = apply_mxfp8(self.model)
            self.print(f"MXFP8: {n_fp8} linear layers run the block-scaled e4m3 GEMM")
        if self.config.nvfp4:
            from archscale_b200.models.layers import apply_nvfp4
            n_fp4 = apply_nvfp4(self.model)
            self.print(f"NVFP4: {n_fp4} linear layers run the block-scaled e2m1 GEMM")
        if self.config.tp_size > 1:
            from archscale_b200.parallel import tp as tp_mod
            tp_mod.apply_tensor_parallel(self.model, mesh)
            if fused_comm:
                # all-gather→GEMM and GEMM→reduce-scatter over peer memory for the column- / row-parallel layers
                tp_mod.enable_fused_layers(self.model, mesh, device, p.micro_batch_size * self.config.block_size)
        if self.config.ep_size > 1:
            from archscale_b200.parallel import ep as ep_mod
            ep_mod.attach(self.model, mesh)
        if p.activation_checkpointing:
            from archscale_b200.parallel.act_ckpt import apply_activation_checkpointing
            apply_activation_checkpointing(self.model)
        self.engine = FSDPEngine(self.model, mesh, unit_classes=(Block,), param_dtype=compute_dtype,
                                 device=device, fused_comm=fused_comm)
        self.print(f"model {p.model_name}: {self.n_params_actual:,} parameters, built in {time.perf_counter() - t0:.1f}s")
        self.optimizer = self._build_optimizer()
        if p.cpu_offload:
            # --offloading / --fsdp_save_mem: fp32 master and optimizer-state shards wait in pinned host memory between steps
            self.engine.enable_cpu_offload([self.optimizer.m, self.optimizer.v])
            self.engine.offload_states()
        self.state = {"iter_num": 0, "step_count": 0}
        self.loss_func = (FusedLinearCrossEntropyLoss(label_smoothing=p.label_smoothing) if p.use_flce_loss
                          else FusedCrossEntropyLoss(label_smoothing=p.label_smoothing))
        self.logger = lu.MetricLogger(p.out_dir if not quiet else None, wandb_project, p.name,
                                      use_wandb=bool(wandb_project) and not quiet, use_mlflow=use_mlflow, rank=mesh.rank)
        self.monitor = SpeedMonitor(get_flops_available(device), window_size=2, world_size=mesh.world,
                                    log_fn=self.logger.log_dict if self.rank0 else None)
        self.train_data_dir, self.val_data_dir = train_data_dir, val_data_dir
        if load_dir is not None:
            path = load_dir if load_dir.endswith(".pth") else ckpt.latest_ckpt_in_dir(load_dir)
            self.print(f"loading weights from {path}")
            self.engine.load_full_state_dict(ckpt.load_anywhere(path)["model"])
        self.resumed = False
        rp = ckpt.find_resume_path(resume, p.out_dir)
        if rp:
            self.print(f"resuming from {rp}")
            self.load_checkpoint(rp)
            self.resumed = True

    # ------------------------------------------------------------------ utils
    def _health(self):
        """Heartbeat / abort store shared by the ranks (multi-rank runs only; ARCHSCALE_B200_HEALTH=0 disables)."""
        if self.mesh.world <= 1 or os.environ.get("ARCHSCALE_B200_HEALTH", "1") == "0":
            return None
        try:
            import torch.distributed as dist
            from archscale_b200.utils.health import Heartbeat
            port = int(os.environ.get("MASTER_PORT", "29500")) + 7
            store = dist.TCPStore(os.environ.get("MASTER_ADDR", "127.0.0.1"), port, self.mesh.world, self.mesh.rank == 0,
                                  wait_for_workers=False)
            return Heartbeat(store, self.mesh.rank, self.mesh.world,
                             stale_after_s=float(os.environ.get("ARCHSCALE_B200_HEARTBEAT_STALE_S", "600")))
        except Exception as e:  # noqa: BLE001 - failure detection must never stop a healthy run
            self.print(f"health store unavailable ({e!r}); continuing without heartbeats")
            return None

    def print(self, *a) -> None:
        if self.rank0 and not self.quiet:
            print(*a, flush=True)

    def _build_optimizer(self) -> ShardedOptimizer:
        p, tc = self.plan, self.plan.train_config
        if not p.mup:
            return ShardedOptimizer(self.engine, lr=p.learning_rate, betas=(p.beta1, p.beta2), eps=p.eps,
                                    weight_decay=p.weight_decay, algorithm="adamw", split_groups=False)
        vector_decay = p.weight_decay if p.original_mup else 0.0
        if "muonball" in tc:
            from archscale_b200.optim.muon_ball import ShardedMuonBall
            return ShardedMuonBall(self.engine, lr=p.learning_rate, betas=(p.beta1, p.beta2), eps=p.eps,
                                   vector_weight_decay=vector_decay, mu=p.muon_beta)
        if "muon" in tc:
            return ShardedOptimizer(self.engine, lr=p.learning_rate, betas=(p.beta1, p.beta2), eps=p.eps,
                                    weight_decay=p.weight_decay, vector_weight_decay=vector_decay, weight_lr_mult=1.0,
                                    algorithm="muonh" if "muonh" in tc else "muon", mu=p.muon_beta, nesterov=True,
                                    adjust_lr="spectral_norm", ns_epsilon=p.eps)
        if "hadam" in tc:
            # AdamW(0.8, 0.95, eps 1e-10) for vectors + NAdam(beta1, beta2, eps) at lr·weight_lr_scale for the weights
            return ShardedOptimizer(self.engine, lr=p.learning_rate, betas=(p.beta1, p.beta2), eps=p.eps,
                                    weight_decay=p.weight_decay, vector_weight_decay=vector_decay,
                                    weight_lr_mult=self.matrix_lr_mult(), algorithm="hadam",
                                    vector_betas=(0.8, 0.95), vector_eps=1e-10)
        return ShardedOptimizer(self.engine, lr=p.learning_rate, betas=(p.beta1, p.beta2), eps=p.eps,
                                weight_decay=p.weight_decay, vector_weight_decay=vector_decay,
                                weight_lr_mult=self.matrix_lr_mult(), algorithm="adamw")

    def matrix_lr_mult(self) -> float:
        """LR multiplier of the weight-matrix class (`pretrain.py:565-592,880-892`): 1 under Muon (the optimizer keeps the
        update RMS itself), ``d0/depth`` otherwise, times ``weight_lr_scale`` for the two-optimizer runs."""
        p, tc = self.plan, self.plan.train_config
        if not p.mup:
            return 1.0
        mult = 1.0 if "muon" in tc else self.base_hps.d0 / p.depth
        if "hadam" in tc or "muonball" in tc:
            mult *= p.weight_lr_scale
        return mult

    # ------------------------------------------------------------------ data
    def _sample_stream(self, data_dir: str, block: int, split: str, seed: int = 12345):
        p, mesh = self.plan, self.mesh
        if data_dir == "synthetic":
            ln = (1500.0, 1.0) if p.use_cu_seqlen else None
            return SyntheticTokens(self.config.vocab_size, block, seed=0 if split == "train" else 1,
                                   rank=mesh.data_rank, eos_token_id=self.config.eos_token_id if ln else None,
                                   doc_len_lognormal=ln, doc_len_clip=(64, p.seq_len))
        cfg = p.train_data_config if split == "train" else p.val_data_config
        datasets = []
        for prefix, _ in cfg:
            files = sorted(glob.glob(os.path.join(data_dir, f"{prefix}*.bin")))
            random.Random(seed).shuffle(files)
            n_chunks = p.data_chunks if split == "train" else math.ceil(8 / p.nodes)
            datasets.append(PackedDataset(files, n_chunks=n_chunks, block_size=block, shuffle=split == "train",
                                          seed=seed + mesh.data_rank, num_processes=mesh.data_world,
                                          process_rank=mesh.data_rank, drop_last=n_chunks <= 8))
        if not datasets or not datasets[0]._filenames:
            raise RuntimeError(f"No data found at {data_dir}. Did you create the dataset?")
        w = [x for _, x in cfg]
        return iter(CombinedDataset(datasets, seed=seed, weights=[x / sum(w) for x in w]))

    def train_loader(self, skip_batches: int = 0) -> PinnedBatchLoader:
        p = self.plan
        stream = self._sample_stream(self.train_data_dir, p.seq_len + 1, "train")
        if skip_batches:
            stream.skip(skip_batches * p.micro_batch_size)
        return PinnedBatchLoader(stream, p.micro_batch_size)

    def val_loader(self) -> Optional[PinnedBatchLoader]:
        if not self.val_data_dir:
            return None
        p = self.plan
        stream = self._sample_stream(self.val_data_dir, p.num_extrapol * p.seq_len + 1, "validation")
        return PinnedBatchLoader(stream, -(p.micro_batch_size // -2))

    # ------------------------------------------------------------------ checkpoint
    def save_checkpoint(self, path: Optional[str] = None) -> str:
        p = self.plan
        path = path or os.path.join(p.out_dir, ckpt.ckpt_name(self.state["iter_num"]))
        state = {
            "model": self.engine.full_state_dict(),
            "optimizer": self.optimizer.state_dict(),
            "hparams": {k: v for k, v in dataclasses.asdict(p).items() if isinstance(v, (int, float, str, bool))},
            "iter_num": self.state["iter_num"],
            "step_count": self.state["step_count"],
            "config": self.config.to_dict(),
            "rng": {"torch": torch.get_rng_state(), "python": random.getstate()},
        }
        ckpt.save_anywhere(path, state, rank=self.mesh.rank)
        return path

    def load_checkpoint(self, path: str) -> None:
        st = ckpt.load_anywhere(path)
        self.engine.load_full_state_dict(st["model"])
        if st.get("optimizer"):
            self.optimizer.load_state_dict(st["optimizer"])
        self.state["iter_num"], self.state["step_count"] = st["iter_num"], st["step_count"]
        if "rng" in st:
            torch.set_rng_state(st["rng"]["torch"])
            random.setstate(st["rng"]["python"])
        # every rank reads the same consolidated file; ranks other than 0 got {} from optimizer.state_dict()

    # ------------------------------------------------------------------ one micro-step
    def forward_backward(self, batch_dev: torch.Tensor, is_code: bool = False, accum: int = 1):
        p = self.plan
        T = self.config.block_size
        if p.use_cu_seqlen and batch_dev.shape[0] > 1:
            batch_dev = batch_dev.reshape(1, -1)
        input_ids = batch_dev[:, :T].contiguous()
        targets = batch_dev[:, 1:T + 1].contiguous()
        tp = self.mesh.tp
        if tp > 1:
            # the model returns this rank's chunk of the tokens; the global loss is the mean of the tp ranks' means
            from archscale_b200.parallel.tp import token_slice
            targets = token_slice(targets, tp, self.mesh.tp_rank).contiguous()
        drop = p.code_dropout if is_code else 0.0        # residual dropout on batches that hold code samples
        if p.use_flce_loss:
            out = self.model(input_ids, use_flce_loss=True, residual_dropout=drop)
            loss = self.loss_func(out.logits, out.weight, targets)
        else:
            loss = self.loss_func(self.model(input_ids, residual_dropout=drop).logits, targets)
        back = loss / tp if tp > 1 else loss
        bal = None
        if self.config.moe:
            bal = self.model.aux_loss
            back = back + bal
        gates = getattr(self.model, "lc_gate_hist", None)
        if gates:
            # layer-configurator models: push the kept-token fraction of every layer towards the budget
            # (`pretrain.py:910-924` of the reference)
            from archscale_b200.ops.moe import activation_budget_loss
            probs = torch.stack([g.squeeze(-1) for g in gates], dim=1)             # (B, L, T)
            self.last_budget_loss = activation_budget_loss(probs, tau=self.config.lc_budget_tau,
                                                           lambda_budget=self.config.lc_budget_lambda)
            back = back + self.last_budget_loss
            self.last_budget_loss = self.last_budget_loss.detach()
        self.engine.backward(back / accum if accum != 1 else back)
        loss = loss.detach()
        if tp > 1:
            loss = loss / tp
            du.all_reduce_sum(loss, group=self.mesh.tp_group)
        return loss, (bal.detach() if isinstance(bal, torch.Tensor) else None)

    def optimizer_step(self, lr: float, hparams: Optional[Dict[str, Dict[str, Any]]] = None):
        if self.mesh.tp > 1:
            from archscale_b200.parallel.tp import sync_replicated_grads
            sync_replicated_grads(self.engine, self.mesh)
        gn, coef = self.engine.clip_grad_norm_(self.plan.grad_clip, defer=True)      # the optimizer applies the coefficient
        kw: Dict[str, Any] = {"grad_scale": coef}
        if hparams is not None:
            hv, hm = hparams["vector"], hparams["matrix"]
            kw.update(weight_decay=hm["weight_decay"], vector_weight_decay=hv["weight_decay"], betas=hm["betas"],
                      eps=hm["eps"], vector_betas=hv["betas"], vector_eps=hv["eps"])
        self.optimizer.step(lr=lr, **kw)
        self.optimizer.zero_grad()
        self.engine.offload_states()
        return gn

    # ------------------------------------------------------------------ loops
    def fit(self) -> None:
        p, state = self.plan, self.state
        tc = p.train_config
        # every evaluation reads the same leading batches of the validation stream (a fresh loader per call, as the
        # reference re-iterates its DataLoader, `pretrain.py:1040`), so val_loss values are comparable between evals
        has_val = bool(self.val_data_dir)
        if has_val:
            self.validate(sanity_check="validation" not in tc)
        if "validation" in tc:
            return
        # MFU counts the parameters of the model that runs (non-embedding; routed experts by the fraction a token visits).
        # The analytic law of the reference (`lit_gpt/config.py:232-265`) assumes the registry shape and is printed beside it.
        n_law = get_parameters_count(p.model_name, p.depth, self.config, tc) if self.config.ar else float("nan")
        n_params = matmul_parameter_count(self.model, self.config, tp=self.mesh.tp, ep=self.mesh.ep)
        flops_per_batch = estimate_flops(self.config, n_params) * p.micro_batch_size / max(self.mesh.tp, 1)
        self.print(f"parameters in the FLOPs estimate: {n_params:,.0f} (non-embedding, counted); analytic law: {n_law:,.0f}; "
                   f"all parameters: {self.n_params_actual:,}; "
                   f"TFLOPs / micro-batch (all ranks): {flops_per_batch * self.mesh.world / 1e12:.2f}")
        world = self.mesh.data_world
        tokens_per_iter = p.micro_batch_size * self.config.block_size
        max_iters = p.train_tokens // world // tokens_per_iter
        if self.max_steps is not None:
            max_iters = min(max_iters, self.max_steps * p.gradient_accumulation_steps)
        warmup_iters = p.warmup_tokens // world // tokens_per_iter
        accum = p.gradient_accumulation_steps
        ramp = p.bsz_rampup_ratio != 1
        learning_rate = p.learning_rate
        loader = self.train_loader(skip_batches=state["iter_num"] if self.resumed else 0)
        # statistics of a logging step are reduced to scalars on this process; formatting them (and the per-layer hooks) runs
        # on a worker — a spawned process when --logging_multiprocessing is on (`logging_utils.py:92-119` of the reference)
        lu.configure_logging_executor(use_multiprocessing=self.logging_multiprocessing and self.rank0)
        total_t0 = time.perf_counter()
        total_lengths = 0
        timer = DeviceStepTimer()
        timer.start()
        device_time_s = 0.0
        log_iter_interval = p.log_step_interval * accum
        self.model.train()
        batch_info = None
        health = self._health()
        fused = getattr(self.engine, "symm", None) is not None
        check_every = int(os.environ.get("ARCHSCALE_B200_DEVICE_CHECK_EVERY", "1" if fused else "0"))
        guard = health.guard() if health is not None else contextlib.nullcontext()
        with guard:
            for train_data, is_code in loader:
                lu.drain_logging_queue(self.logger.log_dict, self.print)
                if state["iter_num"] >= max_iters:
                    break
                if health is not None:
                    # learn about a failed peer on the host, before launching collectives that would wait for it
                    health.check()
                    health.beat(state["iter_num"])
                is_accumulating = (state["iter_num"] + 1) % accum != 0
                ramp_now = None
                if ramp and not is_accumulating:
                    mult = batch_size_rampup_func(state["iter_num"], max_iters, p.bsz_rampup_ratio)
                    accum = int(p.gradient_accumulation_steps * mult)
                    cur_b = p.micro_batch_size * accum * world * p.seq_len
                    ramp_now = apply_batch_size_scaling(cur_b / self.base_hps.b0, self.base_hps, p.bsz_scaling)
                    # as in the reference (`pretrain.py:825-826`) the peak LR becomes the batch-scaled base value
                    learning_rate = ramp_now["learning_rate"]
                    batch_info = {"grad_accum_steps": accum, "effective_batch_size": cur_b, "batch_multiplier": mult,
                                  "batch_ratio": cur_b / self.base_hps.b0}
                lr = get_lr(state["iter_num"], warmup_iters, max_iters, learning_rate, p.min_lr, tc)
                hp = step_hparams(tc, lr=lr, learning_rate=learning_rate, weight_decay=p.weight_decay,
                                  vector_decay=p.weight_decay if p.original_mup else 0.0,
                                  matrix_lr_mult=self.matrix_lr_mult(), super_mup=p.super_mup, ramp=ramp_now)
                log_now = (state["iter_num"] + 1) % log_iter_interval == 0
                self.model.set_collect_stats(log_now)
                batch_dev = train_data.to(self.device, non_blocking=True)
                loss, bal = self.forward_backward(batch_dev, is_code, accum)
                gn = None
                if not is_accumulating:
                    if check_every and self.device.type == "cuda" and state["step_count"] % check_every == 0:
                        # peer-memory kernels give up a wait after a time limit and return; the status word says so.  Read
                        # it before the optimizer consumes gradients that a timed-out pull left incomplete.
                        from archscale_b200.utils.health import check_device
                        check_device()
                    gn = self.optimizer_step(lr, hp)
                    state["step_count"] += 1
                    if fused and state["step_count"] == 3:
                        # start-up skew (allocation, first launches) is over: a peer that stays silent for this long is gone
                        from archscale_b200.ops import backend
                        secs = float(os.environ.get("ARCHSCALE_B200_PEER_WAIT_S", "5"))
                        backend.require_extension().set_peer_wait_limit_cycles(int(secs * 2e9))
                state["iter_num"] += 1
                total_lengths += train_data.shape[0] * self.config.block_size
                if log_now:
                    timer.stop()
                    device_time_s += timer.elapsed_ms() / 1e3        # the only host sync of the loop
                    timer.start()
                    loss_v = float(loss)
                    if self.device.type == "cuda" and not check_every:
                        from archscale_b200.utils.health import check_device
                        check_device()                                 # the stream is already synchronised here
                    self.monitor.on_train_batch_end(state["iter_num"] * p.micro_batch_size, device_time_s,
                                                    flops_per_batch=flops_per_batch, lengths=total_lengths,
                                                    train_loss=loss_v)
                    elapsed = time.perf_counter() - total_t0
                    remaining = elapsed / max(state["iter_num"], 1) * (max_iters - state["iter_num"]) / 3600
                    self.print(f"iter {state['iter_num']} step {state['step_count']}: loss {loss_v:.4f}, lr {lr:.3e}, "
                               f"device time {device_time_s:.1f}s, remaining {remaining:.2f} h")
                    if gn is not None:
                        payload = lu.build_logging_payload(
                            state["iter_num"], state["step_count"], gn, p.grad_clip, model=self.model,
                            optimizer_stats={"betas": self.optimizer.betas, "eps": self.optimizer.eps, "weight_lr": lr,
                                             "vector_lr": lr, "weight_decay": self.optimizer.weight_decay},
                            bal_loss=bal, batch_info=batch_info, vector_names=VECTOR_NAMES)
                        if self.rank0:
                            lu.submit_logging_task(payload)
                if not is_accumulating and has_val and state["step_count"] % p.eval_step_interval == 0:
                    self.validate()
                if not is_accumulating and state["step_count"] % p.save_step_interval == 0:
                    self.print(f"saving checkpoint to {self.save_checkpoint()!r}")
        loader.close()
        if state["iter_num"] >= max_iters and self.max_steps is None:
            if has_val:
                self.validate()
            self.print(f"saving final checkpoint to {self.save_checkpoint()!r}")
        lu.wait_for_logging_tasks(self.logger.log_dict, self.print)
        if self.device.type == "cuda":
            self.print(f"peak memory: {torch.cuda.max_memory_allocated(self.device) / 1e9:.2f} GB")

    @torch.no_grad()
    def validate(self, val_loader=None, sanity_check: bool = False) -> torch.Tensor:
        p = self.plan
        t0 = time.perf_counter()
        self.model.eval()
        iters = 2 if sanity_check else p.eval_iters
        own_loader = val_loader is None
        if own_loader:
            val_loader = self.val_loader()
        losses = torch.zeros(iters, p.num_extrapol, device=self.device)
        accs = None if p.use_flce_loss else torch.zeros(iters, p.num_extrapol, device=self.device)
        seen = 0
        for k in range(iters):
            try:
                val_data, _ = next(val_loader)
            except StopIteration:
                break
            seen += 1
            val_data = val_data.to(self.device, non_blocking=True)
            for i in range(p.num_extrapol):
                length = (i + 1) * p.seq_len
                ids, tgt = val_data[:, :length].contiguous(), val_data[:, 1:length + 1].contiguous()
                if p.use_flce_loss:
                    out = self.model(ids, use_flce_loss=True)
                    losses[k, i] = self.loss_func(out.logits, out.weight, tgt)
                else:
                    logits = self.model(ids).logits
                    losses[k, i] = self.loss_func(logits, tgt)
                    accs[k, i] = (logits.argmax(dim=-1) == tgt).float().mean()
        if own_loader:
            val_loader.close()
        # average over the batches actually read (a short validation set must not average in zeros)
        losses = losses[:max(seen, 1)]
        if accs is not None:
            accs = accs[:max(seen, 1)]
        out = losses.mean(0)
        if "v2scale" in p.train_config and self.mesh.world > 1:
            du.all_reduce_sum(out)
            out /= self.mesh.world
        self.model.train()
        dt = time.perf_counter() - t0
        self.monitor.eval_end(dt)
        if sanity_check:
            return out
        vals = out.tolist()
        for i, v in enumerate(vals):
            self.print(f"step {self.state['iter_num']}: val loss@{i + 1}x {v:.4f}, val time: {dt * 1000:.2f}ms")
            log = {f"metric/val_loss@{i + 1}x": v, f"metric/val_ppl@{i + 1}x": math.exp(min(v, 50.0)),
                   "total_tokens": self.config.block_size * (self.state["iter_num"] + 1) * p.micro_batch_size * self.mesh.world}
            if accs is not None:
                log[f"metric/val_acc_seq@{i + 1}x"] = float(accs.mean(0)[i])
            self.logger.log_dict(log, self.state["step_count"])
        du.barrier()
        return out


# =====================================================================================
def setup(train_data_dir: str = "data/redpajama_sample", val_data_dir: Optional[str] = None,
          load_dir: Optional[str] = None, resume: Union[bool, str] = False, train_model: Optional[str] = None,
          train_name: str = "scaling_mup_tie_rbase_prolong_varlen", depth: int = 16, max_tokens: Optional[float] = None,
          ctx_len: Optional[int] = None, swa_len: Optional[int] = None, data_mixture: Optional[str] = None,
          fsdp_save_mem: bool = False, use_mlflow: bool = False, save_step: Optional[int] = None,
          base_hps: Optional[BaseHyperparameters] = None, micro_bsz: int = 2, total_bsz: Optional[int] = None,
          yarn_scale: float = 1.0, sparsity: int = 1, top_k: int = 2, use_flce: Optional[bool] = None,
          norm_class: Optional[str] = None, fp8: bool = False, fp4: bool = False, post_norm: Optional[bool] = None,
          bramp_ratio: Optional[int] = None, aux_style: Optional[str] = None, aux_gamma: Optional[float] = None,
          fsdp2: bool = False, num_extrp: Optional[int] = None, offloading: bool = False, ortho_init: bool = False,
          diag_init: bool = False, maxfan_init: bool = False, act_ckpt: bool = False,
          share_expert: Optional[bool] = None, global_aux: Optional[bool] = None, sqrt_gate: Optional[bool] = None,
          head_init_std: Optional[float] = 0.02, logging_multiprocessing: bool = True, ar: Optional[int] = None,
          wandb_project: Optional[str] = None,
          # --- additions ---
          tp: int = 1, ep: int = 1, dp_replicate: int = 1, precision: str = "bf16", fused_comm: bool = False,
          max_steps: Optional[int] = None, config_overrides: Optional[Dict[str, Any]] = None,
          return_trainer: bool = False, quiet: bool = False):
    """Same keyword surface as the reference ``setup()`` plus the parallelism additions.

    ``fsdp2`` is accepted for compatibility: this engine is always the sharded one.
    ``dp_replicate`` > 1 gives hybrid sharding (replicate across nodes, shard inside)."""
    # fp32 matmuls (the chunk-parallel products of the SSD scan and the gated delta rule, their backward) on the TF32 tensor
    # cores, as the reference sets at its entry point (`pretrain.py:1329`); here for every caller of setup()
    torch.set_float32_matmul_precision("high")
    base_hps = base_hps or BaseHyperparameters()
    for flag, kind in ((ortho_init, "ortho"), (diag_init, "diag"), (maxfan_init, "maxfan")):
        if flag:
            init_utils.set_default_init(kind)
    du.init_process_group()
    world = du.world_size()
    local_world = int(os.environ.get("LOCAL_WORLD_SIZE", world))
    if torch.cuda.is_available():
        device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0)))
        torch.cuda.set_device(device)
    else:
        device = torch.device("cpu")
    mesh = build_mesh(dp=dp_replicate, tp=tp, ep=ep)
    plan = make_plan(train_model=train_model, train_name=train_name, depth=depth, max_tokens=max_tokens,
                     ctx_len=ctx_len, swa_len=swa_len, data_mixture=data_mixture, fsdp_save_mem=fsdp_save_mem,
                     save_step=save_step, base_hps=base_hps, micro_bsz=micro_bsz, total_bsz=total_bsz,
                     yarn_scale=yarn_scale, sparsity=sparsity, top_k=top_k, use_flce=use_flce, norm_class=norm_class,
                     fp8=fp8, fp4=fp4, post_norm=post_norm, bramp_ratio=bramp_ratio, aux_style=aux_style,
                     aux_gamma=aux_gamma, num_extrp=num_extrp, offloading=offloading, act_ckpt=act_ckpt,
                     share_expert=share_expert, global_aux=global_aux, sqrt_gate=sqrt_gate,
                     head_init_std=head_init_std, ar=ar, load_dir=load_dir, world_size=world,
                     local_world_size=local_world, tp=tp, ep=ep, extra_overrides=config_overrides)
    if mesh.rank == 0:
        ckpt.make_dirs(plan.out_dir)
    trainer = Trainer(plan, mesh, device, train_data_dir, val_data_dir, resume, load_dir, base_hps,
                      use_mlflow=use_mlflow, wandb_project=wandb_project, precision=precision,
                      fused_comm=fused_comm, max_steps=max_steps, quiet=quiet,
                      logging_multiprocessing=logging_multiprocessing)
    if return_trainer:
        return trainer
    trainer.logger.log_hyperparams({**dataclasses.asdict(base_hps),
                                    **{k: v for k, v in dataclasses.asdict(plan).items() if isinstance(v, (int, float))}})
    trainer.fit()
    trainer.logger.close()
    return trainer


# ------------------------------------------------------------------ CLI
def _parse_value(s: str):
    low = s.lower()
    if low in ("true", "false"):
        return low == "true"
    if low in ("none", "null"):
        return None
    for cast in (int, float):
        try:
            return cast(s)
        except ValueError:
            pass
    return s


def parse_cli(argv: List[str]) -> Dict[str, Any]:
    """``--flag value`` / ``--flag=value`` / bare ``--flag`` (true); ``--base_hps.eta0=4e-4`` builds
    the :class:`BaseHyperparameters`; ``--cfg.FIELD=v`` goes to ``config_overrides``."""
    out: Dict[str, Any] = {}
    hps: Dict[str, Any] = {}
    cfg: Dict[str, Any] = {}
    i = 0
    while i < len(argv):
        a = argv[i]
        assert a.startswith("--"), f"unexpected argument {a!r}"
        if "=" in a:
            k, v = a[2:].split("=", 1)
        elif i + 1 < len(argv) and not argv[i + 1].startswith("--"):
            k, v = a[2:], argv[i + 1]
            i += 1
        else:
            k, v = a[2:], "true"
        i += 1
        val = _parse_value(v)
        if k.startswith("base_hps."):
            hps[k.split(".", 1)[1]] = val
        elif k.startswith("cfg."):
            cfg[k.split(".", 1)[1]] = val
        else:
            out[k] = val
    if hps:
        out["base_hps"] = BaseHyperparameters(**hps)
    if cfg:
        out["config_overrides"] = cfg
    return out


def main(argv: Optional[List[str]] = None) -> None:
    torch.set_float32_matmul_precision("high")
    setup(**parse_cli(sys.argv[1:] if argv is None else argv))


if __name__ == "__main__":
    main()
