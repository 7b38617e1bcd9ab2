"""Headline benchmark: training throughput (tokens/s, whole job) of the depth-16 dense GQA
transformer with the MuonH optimizer (or the depth-8 64-expert MoE with ``--config moe``) on N GPUs
of one node, synthetic uniform-random tokens, random-init weights, bf16 compute.

    python bench.py --gpus 1 --steps 10 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 8 --steps 10 --warmup 3

One step = forward + backward + gradient clip + optimizer step on one micro-batch per GPU
(8×4096 tokens for the dense config, 16×4096 for the MoE config).  Rank 0 prints one JSON line.
``value`` is device-timed (CUDA events, max over ranks) with inputs already on the device;
``e2e`` repeats the measurement through the public trainer API with a pinned-host → device copy
of every step's tokens and a device → host read of every step's loss inside the timed region.
``--impl reference`` would run the unmodified reference; it cannot be installed offline (no
build metadata, and its imports lightning / transformer_engine / sonicmoe / mamba_ssm are absent),
so that arm reports ``unavailable``.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

CONFIGS = {
    "dense": dict(
        name="dense GQA d16 (d_model 2048, 16q/4kv heads, head_dim 128, QK-RMSNorm, SwiGLU 5632, vocab 32000), muP++ MuonH",
        train_model="transformer_gqa4", depth=16, train_name="scaling_mup_muonh_qknorm", micro_bsz=8, ctx_len=4096,
        overrides={"intermediate_size": 5632}, sparsity=1, top_k=2),
    "moe": dict(
        name="MoE d8 (d_model 1024, 8q/2kv heads, 64 routed experts hidden 256 + shared 2048, top-8, SqrtGate, "
             "global aux 0.01), muP++ MuonH",
        train_model="transformer_gqa4_h2_moe", depth=8, train_name="scaling_mup_muonh_qknorm", micro_bsz=16, ctx_len=4096,
        overrides={"n_head": 8, "n_query_groups": 2, "n_routed_experts": 64, "router_top_k": 8,
                   "moe_intermediate_size": 256, "shared_intermediate_size": 2048},
        sparsity=8, top_k=8, share_expert=True, sqrt_gate=True, global_aux=True, aux_gamma=0.01),
    "d24": dict(
        name="dense GQA d24 (d_model 3072, 24q/8kv heads, head_dim 128, SwiGLU 8192, vocab 32000), muP++ MuonH; run it with "
             "--fp8 --tp 2 --act-ckpt for the MXFP8 tensor-parallel configuration",
        train_model="transformer_gqa4", depth=24, train_name="scaling_mup_muonh_qknorm", micro_bsz=4, ctx_len=8192,
        overrides={"n_embd": 3072, "n_head": 24, "n_query_groups": 8, "intermediate_size": 8192}, sparsity=1, top_k=2),
    "phi4": dict(
        name="SambaY 3.8B phi4miniflash_d32 (d_model 2560, 40q/20kv heads, head_dim 64, Mamba-1 + SWA 512 + YOCO + GMU, "
             "differential attention, LayerNorm, vocab 200064, tied embeddings), packed 8192-token rows",
        train_model="phi4miniflash", depth=32, train_name="scaling_mup_muonh_tie", micro_bsz=1, ctx_len=8192,
        overrides={}, sparsity=1, top_k=2),
    "gdny": dict(
        name="GDN-Y d16 (Gated DeltaNet + YOCO decoder-hybrid-decoder), muP++ MuonH",
        train_model="gdny", depth=16, train_name="scaling_mup_muonh", micro_bsz=8, ctx_len=4096,
        overrides={}, sparsity=1, top_k=2),
    "mambay2": dict(
        name="Mamba-2-Y d16 (Mamba-2 SSD + YOCO decoder-hybrid-decoder), muP++ MuonH",
        train_model="mambay2", depth=16, train_name="scaling_mup_muonh", micro_bsz=8, ctx_len=4096,
        overrides={}, sparsity=1, top_k=2),
    "sambay": dict(
        name="SambaY d16 (Mamba-1 + SWA + YOCO + GMU), muP++ MuonH",
        train_model="sambay", depth=16, train_name="scaling_mup_muonh", micro_bsz=8, ctx_len=4096,
        overrides={}, sparsity=1, top_k=2),
}

CLOCK_QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
               "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
               "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")


class ClockSampler:
    """``nvidia-smi`` sampling in a child process while the timed region runs (read-only)."""

    def __init__(self, gpu_index: int) -> None:
        self.path = tempfile.mktemp(suffix=".csv")
        self.proc = None
        self.gpu_index = gpu_index

    def start(self) -> None:
        try:
            self.fh = open(self.path, "w")
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={CLOCK_QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.gpu_index)], stdout=self.fh,
                                         stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.fh.close()
        sm, mx, reasons = [], [], set()
        try:
            for line in open(self.path):
                f = [x.strip() for x in line.split(",")]
                if len(f) < 9:
                    continue
                try:
                    sm.append(float(f[1]))
                    mx.append(float(f[2]))
                except ValueError:
                    continue
                for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except OSError:
            pass
        if sm:
            out.update(sm_mhz=statistics.median(sm), sm_max_mhz=max(mx), samples=len(sm))
        out["reasons"] = sorted(reasons)
        return out



def parse_cfg_overrides(items) -> dict:
    """``FIELD=VALUE`` strings → Config overrides: true / false, integers and floats are converted, anything else stays a string."""
    out = {}
    for item in items:
        key, sep, val = item.partition("=")
        if not sep or not key:
            raise ValueError(f"--cfg expects FIELD=VALUE, got {item!r}")
        low = val.lower()
        if low in ("true", "false"):
            out[key] = low == "true"
            continue
        for conv in (int, float):
            try:
                out[key] = conv(val)
                break
            except ValueError:
                pass
        else:
            out[key] = val
    return out

def run_ours(args) -> None:
    import torch
    import torch.distributed as dist

    from archscale_b200.ops import backend
    from archscale_b200.train.pretrain import setup
    from archscale_b200.utils.speed_monitor import estimate_flops, matmul_parameter_count, measured_peaks

    world = int(os.environ.get("WORLD_SIZE", "1"))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}; launch with torch.distributed.run"
    c = CONFIGS[args.config]
    os.environ.setdefault("LIGHTNING_ARTIFACTS_DIR", os.path.join(tempfile.gettempdir(), "archscale_b200_bench"))
    ep = world if (args.config == "moe" and world > 1 and not args.no_ep) else 1
    overrides = dict(c["overrides"])
    overrides.update(parse_cfg_overrides(args.cfg))
    kwargs = dict(train_data_dir="synthetic", train_model=c["train_model"], depth=c["depth"], train_name=c["train_name"],
                  micro_bsz=c["micro_bsz"], ctx_len=c["ctx_len"], total_bsz=(world // max(args.tp, 1)) * c["micro_bsz"] * c["ctx_len"],
                  max_tokens=1e12, use_flce=True, sparsity=c["sparsity"], top_k=c["top_k"],
                  config_overrides=overrides, ep=ep, tp=args.tp, fused_comm=args.fused_comm, fp8=args.fp8, fp4=args.fp4,
                  act_ckpt=args.act_ckpt, return_trainer=True, quiet=True)
    for k in ("share_expert", "sqrt_gate", "global_aux", "aux_gamma"):
        if k in c:
            kwargs[k] = c[k]
    trainer = setup(**kwargs)
    trainer.quiet = True
    dev = trainer.device
    cfg = trainer.config
    mb, T = c["micro_bsz"], c["ctx_len"]
    tokens_per_step = (world // max(args.tp, 1)) * mb * T      # tensor-parallel peers share a micro-batch
    lr = trainer.plan.learning_rate

    g = torch.Generator().manual_seed(0 * 1000003 + trainer.mesh.data_rank)
    n_batches = args.steps + args.warmup
    host_batches = [torch.randint(0, cfg.vocab_size, (mb, T + 1), generator=g).pin_memory() for _ in range(min(n_batches, 8))]
    dev_batches = [b.to(dev) for b in host_batches]

    def step_dev(i):
        loss, _ = trainer.forward_backward(dev_batches[i % len(dev_batches)])
        trainer.optimizer_step(lr)
        return loss

    def sync_all():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        sync_all()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(steps):
            fn(i)
        e1.record()
        sync_all()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms) / steps

    for i in range(args.warmup):
        step_dev(i)
    sampler = ClockSampler(int(os.environ.get("LOCAL_RANK", "0")))
    if trainer.mesh.rank == 0:
        sampler.start()
    backend.reset_launches()
    ms_per_step = timed(step_dev, args.steps)
    launches = backend.launches()
    clocks = sampler.stop() if trainer.mesh.rank == 0 else {}

    # end to end: pinned host tokens → device every step, loss read back every step
    h2d = mb * (T + 1) * 8
    losses = []

    def step_e2e(i):
        batch = host_batches[i % len(host_batches)].to(dev, non_blocking=True)
        loss, _ = trainer.forward_backward(batch)
        trainer.optimizer_step(lr)
        losses.append(float(loss))        # device → host read of the step's result

    e2e_ms = timed(step_e2e, args.steps)

    phases = None
    if args.phases:
        # forward+backward vs optimizer step, device-timed separately (after the headline measurement)
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        fb = op = 0.0
        for i in range(args.steps):
            sync_all()
            ev[0].record()
            trainer.forward_backward(dev_batches[i % len(dev_batches)])
            ev[1].record()
            trainer.optimizer_step(lr)
            ev[2].record()
            torch.cuda.synchronize()
            fb += ev[0].elapsed_time(ev[1])
            op += ev[1].elapsed_time(ev[2])
        phases = {"forward_backward_ms": fb / args.steps, "optimizer_step_ms": op / args.steps}
    if args.kernel_table > 0:
        from torch.profiler import ProfilerActivity, profile
        sync_all()
        if trainer.mesh.rank == 0:
            with profile(activities=[ProfilerActivity.CUDA]) as prof:
                step_dev(0)
                torch.cuda.synchronize()
            rows = sorted(prof.key_averages(), key=lambda e: -e.device_time_total)
            tot = sum(e.device_time_total for e in rows)
            print(f"kernel table: {tot / 1e3:.2f} ms of device time over {sum(e.count for e in rows)} launches in one step "
                  f"(step {ms_per_step:.2f} ms)", file=sys.stderr)
            for e in rows[:args.kernel_table]:
                print(f"{e.device_time_total / 1e3:9.3f} ms {100 * e.device_time_total / tot:5.1f}% x{e.count:5d}  {e.key[:120]}", file=sys.stderr)
        else:
            step_dev(0)
        sync_all()
    status = backend.load_extension().device_status() if backend.load_extension() is not None else 0

    # MFU in the reference's convention (3·(2·N·T + attention over the full T×T square) per sequence, peak 2.25e15), but with N
    # counted from the model that ran (non-embedding, routed experts by the fraction a token visits) instead of the analytic
    # law, which assumes a 4·d_model MLP and over-counts the 5632-wide benchmark shape.
    n_flops = matmul_parameter_count(trainer.model, cfg, include_head=False, tp=max(args.tp, 1), ep=ep)
    n_flops_head = matmul_parameter_count(trainer.model, cfg, include_head=True, tp=max(args.tp, 1), ep=ep)
    flops_step = estimate_flops(cfg, n_flops) * mb
    flops_step_head = estimate_flops(cfg, n_flops_head) * mb
    pk = measured_peaks(ROOT)
    if trainer.mesh.rank == 0:
        value = tokens_per_step / (ms_per_step / 1e3)
        out = {
            "metric": "train tokens/sec (whole job; per GPU = value / n_gpus), device-timed, max over ranks",
            "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "nvfp4 linears (bf16 elsewhere)" if args.fp4 else "mxfp8 linears (bf16 elsewhere)" if args.fp8 else "bf16", "data": "synthetic uniform-random token ids (seed 0), random-init weights",
            "tokens_per_sec_per_gpu": value / world,
            "mfu": flops_step / max(args.tp, 1) / (ms_per_step / 1e3) / 2.25e15,   # per GPU: tp peers share a micro-batch
            "mfu_with_lm_head": flops_step_head / max(args.tp, 1) / (ms_per_step / 1e3) / 2.25e15,
            "frac_of_sustained_bf16": flops_step_head / max(args.tp, 1) / (ms_per_step / 1e3) / (pk["bf16_tflops_sustained"] * 1e12),
            "mfu_note": f"N = {n_flops:,.0f} non-embedding parameters of the shape that ran ({n_flops_head:,.0f} with lm_head); "
                        f"sustained bf16 peak {pk['bf16_tflops_sustained']:.0f} TFLOP/s ({pk['kind']})",
            "config": {"model": c["name"], "global_batch": world * mb, "seq_len": T,
                       "residual_stream": "fp32" if cfg.residual_in_fp32 else "bf16",
                       "parallelism": (f"fsdp{world // max(args.tp, 1)}" if world > 1 else "single") + (f"+ep{ep}" if ep > 1 else "")
                                      + (f"+tp{args.tp}" if args.tp > 1 else ""),
                       "optimizer": "MuonH (Newton-Schulz 5) + AdamW/Adam-H, grad clip 1.0",
                       "l2": "per-step working set (weights + activations, > 10 GB) far exceeds the 126 MB L2; "
                             "no explicit flush",
                       "params": trainer.n_params_actual, "params_in_mfu": n_flops, "final_loss": losses[-1] if losses else None,
                       "device_status": int(status), "fused_comm": bool(args.fused_comm)},
            "clocks": clocks,
            **({"phases": phases} if phases else {}),
            "e2e": {"value": tokens_per_step / (e2e_ms / 1e3), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": 4, "ms_per_step": e2e_ms},
            "gpu_launches": launches,
        }
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_reference(args) -> None:
    ref = os.path.join(ROOT, "baseline", "_ref")
    why = ("reference is not installable offline: its tree has neither setup.py nor pyproject.toml "
           "(pip: 'Directory is not installable'), and its imports lightning, transformer_engine, sonicmoe, "
           "mamba_ssm, causal_conv1d, jsonargparse, blobfile, flash_attn.cute are not in the image")
    if os.path.isdir(ref) and os.listdir(ref):
        why = "baseline/_ref exists but the reference's dependencies (lightning, transformer_engine, sonicmoe) are not importable"
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="dense", choices=sorted(CONFIGS))
    ap.add_argument("--act-ckpt", dest="act_ckpt", action="store_true", help="activation checkpointing per block")
    ap.add_argument("--phases", action="store_true", help="also report forward+backward and optimizer-step times")
    ap.add_argument("--kernel-table", dest="kernel_table", type=int, default=0, metavar="N",
                    help="after the measurement, run one more step under torch.profiler on rank 0 and print the N kernels with "
                         "the largest device time to stderr (shares of the step; not part of any reported number)")
    ap.add_argument("--tp", type=int, default=1, help="tensor-parallel degree (ranks of a tp group share a micro-batch)")
    ap.add_argument("--fp8", action="store_true", help="MXFP8 block-scaled linear layers (dtype is then reported as mxfp8)")
    ap.add_argument("--fp4", action="store_true", help="NVFP4 block-scaled linear layers (dtype is then reported as nvfp4)")
    ap.add_argument("--fused-comm", dest="fused_comm", action="store_true", default=True,
                    help="peer-memory collectives fused with compute (default on more than one GPU)")
    ap.add_argument("--no-fused-comm", dest="fused_comm", action="store_false", help="NCCL collectives (the baseline path)")
    ap.add_argument("--no-ep", dest="no_ep", action="store_true")
    ap.add_argument("--cfg", action="append", default=[], metavar="FIELD=VALUE",
                    help="override a Config field of the benchmarked model (repeatable), e.g. --cfg residual_in_fp32=false")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
