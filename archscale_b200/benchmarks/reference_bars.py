"""This package's kernels timed beside what the reference runs for the same op, on the same tensors and the same GPU.

The reference cannot be run as a whole here (its model imports TransformerEngine, its trainer Lightning), but the kernels
it is built on can: its own Triton files are self-contained (torch / triton / einops only) and are loaded by path from a
checkout named by ``ARCHSCALE_REFERENCE_DIR`` without executing ``lit_gpt/__init__.py``; ``flash_attn`` (the Hopper /
Ampere attention path, `lit_gpt/attention.py:119-120`) and QuACK's sm_100 GEMM (`install.sh:101`) are used when
importable (``fla``'s gated-delta-rule kernel faulted on this GPU and is left out, see :func:`bench_gdn`).  Every row: op, shape, our time, their time, ratio.  A bar that cannot
be loaded prints ``unavailable`` with the reason; nothing here is used by training or by ``bench.py``.

    ARCHSCALE_REFERENCE_DIR=/path/to/ArchScale python -m archscale_b200.benchmarks.reference_bars [rmsnorm rope flce ns gated attn gdn gemm]
"""
from __future__ import annotations

import argparse
import importlib
import json
import os
import sys
import types

import torch

from archscale_b200 import ops
from archscale_b200.benchmarks.kernels import time_ms


def ref_module(name: str):
    """``lit_gpt.<name>`` of the reference checkout, imported under a private package name so that the reference's
    ``__init__`` (which pulls in TransformerEngine) never runs."""
    root = os.environ.get("ARCHSCALE_REFERENCE_DIR")
    if not root or not os.path.isdir(os.path.join(root, "lit_gpt")):
        raise RuntimeError("ARCHSCALE_REFERENCE_DIR does not point at a reference checkout")
    pkg = "_archscale_ref_lit_gpt"
    if pkg not in sys.modules:
        for sub, rel in ((pkg, "lit_gpt"), (pkg + ".ops", "lit_gpt/ops"), (pkg + ".optim", "lit_gpt/optim")):
            m = types.ModuleType(sub)
            m.__path__ = [os.path.join(root, rel)]
            m.__package__ = sub
            sys.modules[sub] = m
    return importlib.import_module(f"{pkg}.{name}")


def _row(res, op, shape, ours_ms, ref_ms, ref_name, **extra):
    r = {"op": op, "shape": shape, "ours_ms": ours_ms, "ref": ref_name, "ref_ms": ref_ms,
         "ours_over_ref_speed": (ref_ms / ours_ms) if (ours_ms and ref_ms) else None, **extra}
    res.append(r)
    print(json.dumps(r), flush=True)


def _try(res, op, fn):
    try:
        fn()
    except Exception as e:  # noqa: BLE001 - a missing bar must not stop the others
        r = {"op": op, "unavailable": f"{type(e).__name__}: {str(e)[:300]}"}
        res.append(r)
        print(json.dumps(r), flush=True)


def bench_rmsnorm(res):
    def run():
        ref = ref_module("rmsnorm")
        for rows, cols in ((32768, 2048), (65536, 1024)):
            x = torch.randn(rows, cols, device="cuda").bfloat16().requires_grad_()
            w = torch.ones(cols, device="cuda", requires_grad=True)
            f_o = lambda: ops.rms_norm(x, w, 1e-5, out_dtype=torch.bfloat16)
            f_r = lambda: ref.rms_norm_fn(x, w, None, eps=1e-5)
            y_o, y_r = f_o(), f_r()
            g = torch.randn_like(y_o)
            _row(res, "rmsnorm fwd", [rows, cols], time_ms(f_o), time_ms(f_r), "lit_gpt/rmsnorm.py (Triton)")
            _row(res, "rmsnorm bwd", [rows, cols], time_ms(lambda: torch.autograd.grad(y_o, (x, w), g, retain_graph=True)),
                 time_ms(lambda: torch.autograd.grad(y_r, (x, w), g, retain_graph=True)), "lit_gpt/rmsnorm.py (Triton)")
    _try(res, "rmsnorm", run)


def bench_rope(res):
    def run():
        ref = ref_module("fused_rotary_embedding")
        B, T, H, G, D = 8, 4096, 16, 4, 128
        q = torch.randn(B, T, H, D, device="cuda").bfloat16().requires_grad_()
        k = torch.randn(B, T, G, D, device="cuda").bfloat16().requires_grad_()
        cos, sin = ops.rope.build_rope_cache(T, D, torch.float32, "cuda")
        f_o = lambda: ops.qk_norm_rope(q, k, None, None, cos, sin)
        f_r = lambda: (ref.apply_rotary_emb(q, cos, sin), ref.apply_rotary_emb(k, cos, sin))
        _row(res, "rope q+k fwd", [B, T, H, G, D], time_ms(f_o), time_ms(f_r), "lit_gpt/fused_rotary_embedding.py (Triton)")
        yo, yr = f_o(), f_r()
        go = [torch.randn_like(t) for t in yo]
        _row(res, "rope q+k bwd", [B, T, H, G, D], time_ms(lambda: torch.autograd.grad(yo, (q, k), go, retain_graph=True)),
             time_ms(lambda: torch.autograd.grad(yr, (q, k), go, retain_graph=True)), "lit_gpt/fused_rotary_embedding.py (Triton)")
    _try(res, "rope", run)


def bench_flce(res):
    def run():
        ref = ref_module("fused_linear_cross_entropy")
        N, H, V = 32768, 2048, 32000
        x = (torch.randn(N, H, device="cuda") * 0.5).bfloat16().requires_grad_()
        w = (torch.randn(V, H, device="cuda") * 0.02).bfloat16().requires_grad_()
        t = torch.randint(0, V, (N,), device="cuda")
        loss_r = ref.FusedLinearCrossEntropyLoss()

        def ours():
            l = ops.fused_linear_cross_entropy(x, w, t)
            torch.autograd.grad(l, (x, w))

        def theirs():
            l = loss_r(x, w, t)
            torch.autograd.grad(l, (x, w))
        _row(res, "linear + cross-entropy fwd+bwd", [N, H, V], time_ms(ours, iters=5), time_ms(theirs, iters=5),
             "lit_gpt/fused_linear_cross_entropy.py (Triton CE + cuBLAS)")
    _try(res, "flce", run)


def bench_ns(res):
    def run():
        ref = ref_module("optim.newton_schulz_triton")
        for shape in ((16, 2048, 2048), (16, 2048, 5632), (64, 512, 1024)):
            G = torch.randn(*shape, device="cuda").bfloat16()
            _row(res, "Newton-Schulz x5 (batched)", list(shape), time_ms(lambda: ops.newton_schulz(G), iters=5),
                 time_ms(lambda: ref.newton_schulz_triton(G), iters=5), "lit_gpt/optim/newton_schulz_triton.py (Triton + cuBLAS)")
    _try(res, "newton_schulz", run)


def bench_gated(res):
    def run():
        ref = ref_module("ops.layernorm_gated")
        rows, cols, gs = 32768, 4096, 512
        x = torch.randn(rows, cols, device="cuda").bfloat16().requires_grad_()
        z = torch.randn(rows, cols, device="cuda").bfloat16().requires_grad_()
        w = torch.ones(cols, device="cuda", requires_grad=True)
        f_o = lambda: ops.gated_rms_norm(x, w, z, 1e-5, gs, False)
        f_r = lambda: ref.rmsnorm_fn(x, w, None, z=z, eps=1e-5, group_size=gs, norm_before_gate=False)
        yo, yr = f_o(), f_r()
        g = torch.randn_like(yo)
        _row(res, "gated RMSNorm fwd", [rows, cols, gs], time_ms(f_o), time_ms(f_r), "lit_gpt/ops/layernorm_gated.py (Triton)")
        _row(res, "gated RMSNorm bwd", [rows, cols, gs], time_ms(lambda: torch.autograd.grad(yo, (x, z, w), g, retain_graph=True)),
             time_ms(lambda: torch.autograd.grad(yr, (x, z, w), g, retain_graph=True)), "lit_gpt/ops/layernorm_gated.py (Triton)")
    _try(res, "gated_rmsnorm", run)


def bench_attn(res):
    def run():
        from flash_attn import flash_attn_func
        import flash_attn
        for (B, T, H, G, D, win) in ((8, 4096, 16, 4, 128, -1), (1, 8192, 20, 10, 64, 511)):
            q = torch.randn(B, T, H, D, device="cuda").bfloat16().requires_grad_()
            k = torch.randn(B, T, G, D, device="cuda").bfloat16().requires_grad_()
            v = torch.randn(B, T, G, D, device="cuda").bfloat16().requires_grad_()
            window = (win, 0) if win >= 0 else (-1, -1)
            f_o = lambda: ops.attention(q, k, v, window=window)
            f_r = lambda: flash_attn_func(q, k, v, causal=True, window_size=window, deterministic=True)
            kq, kk, kv = (t.detach().transpose(1, 2) for t in (q, k, v))
            f_c = lambda: torch.nn.functional.scaled_dot_product_attention(kq, kk, kv, is_causal=True, enable_gqa=True)
            span = T if win < 0 else min(T, win + 1)
            fl = 4.0 * B * H * T * span * D * (0.5 if win < 0 else 1.0)
            to, tr = time_ms(f_o), time_ms(f_r)
            extra = {"ours_tflops": fl / to / 1e9, "ref_tflops": fl / tr / 1e9}
            if win < 0:
                tc = time_ms(f_c)
                extra.update(cudnn_sdpa_ms=tc, cudnn_sdpa_tflops=fl / tc / 1e9)
            _row(res, "attention fwd", [B, T, H, G, D, win], to, tr, f"flash_attn {flash_attn.__version__}", **extra)
            yo, yr = f_o(), f_r()
            g = torch.randn_like(yo)
            to = time_ms(lambda: torch.autograd.grad(yo, (q, k, v), g, retain_graph=True), iters=5)
            tr = time_ms(lambda: torch.autograd.grad(yr, (q, k, v), g, retain_graph=True), iters=5)
            _row(res, "attention bwd", [B, T, H, G, D, win], to, tr, f"flash_attn {flash_attn.__version__} (deterministic)",
                 ours_tflops=2.5 * fl / to / 1e9, ref_tflops=2.5 * fl / tr / 1e9)
    _try(res, "attention", run)


def bench_gdn(res):
    """``fla``'s ``chunk_gated_delta_rule`` (what `lit_gpt/gated_deltanet.py:315-326` calls) is not run: on B200 with
    driver 580 its Triton kernel raised "misaligned address" at the Gated-DeltaNet layer shape (B8 T4096 H6 Dk256 Dv512,
    fla 0.5.1, triton 3.6) and left the CUDA context unusable for the bars after it.  Our own numbers for the op are in
    ``benchmarks.kernels gdn``."""
    r = {"op": "gated_delta_rule", "unavailable": "fla chunk_gated_delta_rule raised a misaligned-address fault on this GPU; not run"}
    res.append(r)
    print(json.dumps(r), flush=True)


def bench_gemm(res):
    def run():
        ext = ops.backend.require_extension()
        try:
            from quack.gemm_interface import gemm as quack_gemm
            name = "QuACK gemm (sm_100 CuTe DSL)"
        except Exception:  # noqa: BLE001
            quack_gemm, name = None, "cuBLAS (torch.matmul)"
        for (M, N, K, what) in ((32768, 3072, 2048, "fwd qkv d16"), (32768, 11264, 2048, "fwd w1 d16"), (8192, 8192, 8192, "square")):
            a, b = torch.randn(M, K, device="cuda").bfloat16(), torch.randn(N, K, device="cuda").bfloat16()
            f_r = (lambda: quack_gemm(a, b.t())) if quack_gemm is not None else (lambda: a @ b.t())
            to, tr = time_ms(lambda: ext.gemm_bf16(a, b, 0, torch.bfloat16, None)), time_ms(f_r)
            _row(res, f"GEMM {what}", [M, N, K], to, tr, name, ours_tflops=2.0 * M * N * K / to / 1e9, ref_tflops=2.0 * M * N * K / tr / 1e9)
    _try(res, "gemm", run)


ALL = {"rmsnorm": bench_rmsnorm, "rope": bench_rope, "flce": bench_flce, "ns": bench_ns, "gated": bench_gated, "attn": bench_attn,
       "gdn": bench_gdn, "gemm": bench_gemm}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("which", nargs="*", default=list(ALL))
    ap.add_argument("--json", default=None)
    a = ap.parse_args()
    res: list = []
    for w in a.which:
        ALL[w](res)
    if a.json:
        json.dump(res, open(a.json, "w"), indent=1)


if __name__ == "__main__":
    main()
