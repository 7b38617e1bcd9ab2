"""Per-kernel microbenchmarks against the measured roofline (``MEASURED_PEAKS.json``) and the
library kernel doing the same op.  CUDA-event timing, warm-up, L2 flushed between iterations.

    python -m archscale_b200.benchmarks.kernels gemm rmsnorm swiglu ce rope attn mamba    # any subset
    python -m archscale_b200.benchmarks.kernels gemm --json out.json
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

from archscale_b200 import ops
from archscale_b200.ops import backend

_flush = None


def flush_l2() -> None:
    global _flush
    if _flush is None:
        _flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    _flush.zero_()


def time_ms(fn, iters: int = 10, warmup: int = 3) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        flush_l2()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    return ts[len(ts) // 2]


def peaks() -> dict:
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    p = os.path.join(root, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "kind": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "kind": "fallback"}


def bench_gemm(res: list) -> None:
    ext = backend.require_extension()
    pk = peaks()
    shapes = [  # (mode, M, N, K, what)
        (0, 32768, 3072, 2048, "fwd qkv d16"), (0, 32768, 2048, 2048, "fwd proj d16"),
        (0, 32768, 11264, 2048, "fwd w1 d16"), (0, 32768, 2048, 5632, "fwd w3 d16"),
        (1, 32768, 2048, 11264, "dgrad w1 d16"), (1, 32768, 5632, 2048, "dgrad w3 d16"),
        (2, 11264, 2048, 32768, "wgrad w1 d16"), (2, 2048, 5632, 32768, "wgrad w3 d16"),
        (0, 4096, 32000, 2048, "flce logits chunk"), (0, 2048, 2048, 2048, "NS XXt 2048"),
        (0, 8192, 8192, 8192, "square 8192"),
    ]
    for mode, M, N, K, what in shapes:
        if mode == 0:
            a, b = torch.randn(M, K, device="cuda").bfloat16(), torch.randn(N, K, device="cuda").bfloat16()
            lib = lambda: a @ b.t()
        elif mode == 1:
            a, b = torch.randn(M, K, device="cuda").bfloat16(), torch.randn(K, N, device="cuda").bfloat16()
            lib = lambda: a @ b
        else:
            a, b = torch.randn(K, M, device="cuda").bfloat16(), torch.randn(K, N, device="cuda").bfloat16()
            lib = lambda: a.t() @ b
        ours = lambda: ext.gemm_bf16(a, b, mode, torch.bfloat16, None)
        t_o, t_l = time_ms(ours), time_ms(lib)
        fl = 2.0 * M * N * K
        res.append({"kernel": "gemm_bf16", "case": what, "mode": mode, "M": M, "N": N, "K": K, "ms": t_o,
                    "tflops": fl / t_o / 1e9, "frac_of_" + pk["kind"] + "_peak": fl / t_o / 1e9 / pk["bf16_tflops"],
                    "cublas_ms": t_l, "cublas_tflops": fl / t_l / 1e9, "vs_cublas": t_l / t_o})
        print(res[-1], flush=True)


def bench_rmsnorm(res: list) -> None:
    pk = peaks()
    for rows, cols, xdt in [(32768, 2048, torch.float32), (32768, 2048, torch.bfloat16), (65536, 1024, torch.float32)]:
        x = torch.randn(rows, cols, device="cuda", dtype=xdt).requires_grad_()
        w = torch.ones(cols, device="cuda", requires_grad=True)
        t_f = time_ms(lambda: ops.rms_norm(x, w, 1e-5, out_dtype=torch.bfloat16))
        y = ops.rms_norm(x, w, 1e-5, out_dtype=torch.bfloat16)
        g = torch.randn_like(y)
        t_b = time_ms(lambda: torch.autograd.grad(y, (x, w), g, retain_graph=True))
        by_f = rows * cols * (x.element_size() + 2)
        by_b = rows * cols * (2 + 2 * x.element_size())
        t_lib = time_ms(lambda: torch.nn.functional.rms_norm(x, (cols,), w, 1e-5).bfloat16())
        res.append({"kernel": "rmsnorm", "rows": rows, "cols": cols, "x": str(xdt), "fwd_ms": t_f,
                    "fwd_gbs": by_f / t_f / 1e6, "fwd_frac_hbm": by_f / t_f / 1e6 / pk["hbm_gbs"], "bwd_ms": t_b,
                    "bwd_gbs": by_b / t_b / 1e6, "bwd_frac_hbm": by_b / t_b / 1e6 / pk["hbm_gbs"], "torch_fwd_ms": t_lib})
        print(res[-1], flush=True)


def bench_swiglu(res: list) -> None:
    pk = peaks()
    rows, I = 32768, 5632
    x = torch.randn(rows, 2 * I, device="cuda").bfloat16().requires_grad_()
    t_f = time_ms(lambda: ops.swiglu_packed(x))
    y = ops.swiglu_packed(x)
    g = torch.randn_like(y)
    t_b = time_ms(lambda: torch.autograd.grad(y, x, g, retain_graph=True))
    by_f, by_b = rows * I * 2 * 3, rows * I * 2 * 5
    a, b = x.detach().chunk(2, dim=-1)
    t_lib = time_ms(lambda: torch.nn.functional.silu(a) * b)
    res.append({"kernel": "swiglu_packed", "rows": rows, "I": I, "fwd_ms": t_f, "fwd_frac_hbm": by_f / t_f / 1e6 / pk["hbm_gbs"],
                "bwd_ms": t_b, "bwd_frac_hbm": by_b / t_b / 1e6 / pk["hbm_gbs"], "torch_fwd_ms": t_lib})
    print(res[-1], flush=True)


def bench_ce(res: list) -> None:
    pk = peaks()
    ext = backend.require_extension()
    rows, V = 4096, 32000
    logits = torch.randn(rows, V, device="cuda").bfloat16()
    tgt = torch.randint(0, V, (rows,), device="cuda")
    t = time_ms(lambda: ext.cross_entropy_fwd_bwd_(logits, tgt, -100, 0.0, 0.0))
    by = rows * V * 2 * 2
    res.append({"kernel": "cross_entropy_fwd_bwd", "rows": rows, "V": V, "ms": t, "frac_hbm_min_traffic": by / t / 1e6 / pk["hbm_gbs"]})
    print(res[-1], flush=True)
    N, H = 32768, 2048
    x = (torch.randn(N, H, device="cuda") * 0.5).bfloat16().requires_grad_()
    w = (torch.randn(V, H, device="cuda") * 0.02).bfloat16().requires_grad_()
    tg = torch.randint(0, V, (N,), device="cuda")

    def flce():
        loss = ops.fused_linear_cross_entropy(x, w, tg)
        loss.backward()
        x.grad = w.grad = None
    t = time_ms(flce, iters=5)
    fl = 3 * 2.0 * N * H * V
    res.append({"kernel": "flce_fwd_bwd", "N": N, "H": H, "V": V, "ms": t, "tflops": fl / t / 1e9,
                "frac_of_" + pk["kind"] + "_peak": fl / t / 1e9 / pk["bf16_tflops"]})
    print(res[-1], flush=True)


def bench_rope(res: list) -> None:
    pk = peaks()
    B, T, H, G, D = 8, 4096, 16, 4, 128
    q = torch.randn(B, T, H, D, device="cuda").bfloat16().requires_grad_()
    k = torch.randn(B, T, G, D, device="cuda").bfloat16().requires_grad_()
    qw = torch.ones(D, device="cuda", requires_grad=True)
    kw = torch.ones(D, device="cuda", requires_grad=True)
    cos, sin = ops.build_rope_cache(T, D, torch.bfloat16, "cuda")
    t_f = time_ms(lambda: ops.qk_norm_rope(q, k, qw, kw, cos, sin, 1e-5))
    by = B * T * (H + G) * D * 2 * 2
    res.append({"kernel": "qknorm_rope_fwd", "shape": [B, T, H, G, D], "ms": t_f, "frac_hbm": by / t_f / 1e6 / pk["hbm_gbs"]})
    print(res[-1], flush=True)


def bench_attn(res: list) -> None:
    pk = peaks()
    for (B, T, H, G, D, win) in [(8, 4096, 16, 4, 128, -1), (1, 8192, 20, 10, 64, 511)]:
        q = torch.randn(B, T, H, D, device="cuda").bfloat16().requires_grad_()
        k = torch.randn(B, T, G, D, device="cuda").bfloat16().requires_grad_()
        v = torch.randn(B, T, G, D, device="cuda").bfloat16().requires_grad_()
        f = lambda: ops.attention(q, k, v, window=(win, 0) if win >= 0 else (-1, -1))
        t_f = time_ms(f)
        o = f()
        g = torch.randn_like(o)
        t_b = time_ms(lambda: torch.autograd.grad(o, (q, k, v), g, retain_graph=True), iters=5)
        span = T if win < 0 else min(T, win + 1)
        fl = 4.0 * B * H * T * span * D * (0.5 if win < 0 else 1.0)
        res.append({"kernel": "attention", "shape": [B, T, H, G, D], "window": win, "native": backend.has("attn_fwd"),
                    "fwd_ms": t_f, "fwd_tflops": fl / t_f / 1e9, "bwd_ms": t_b, "bwd_tflops": 2.5 * fl / t_b / 1e9,
                    "fwd_frac_of_" + pk["kind"] + "_peak": fl / t_f / 1e9 / pk["bf16_tflops"]})
        print(res[-1], flush=True)


def bench_mamba(res: list) -> None:
    """Causal conv1d and selective scan at the Mamba-1 shapes of the SambaY / Phi-4-mini-flash family."""
    pk = peaks()
    for (B, L, Di, what) in [(1, 8192, 5120, "phi4-mini-flash d_inner"), (8, 4096, 4096, "d16-class d_inner")]:
        N = 16
        xz = torch.randn(B, L, 2 * Di, device="cuda").bfloat16()
        x, z = xz[..., :Di], xz[..., Di:]
        w, b = torch.randn(Di, 4, device="cuda"), torch.randn(Di, device="cuda")
        f = lambda: ops.causal_conv1d(x, w, b, activation="silu", channel_last=True)
        t = time_ms(f)
        by = 2 * x.numel() * 2
        res.append({"kernel": "causal_conv1d_fwd", "what": what, "shape": [B, L, Di], "ms": t, "gbs": by / t / 1e6,
                    "frac_of_" + pk["kind"] + "_hbm": by / t / 1e6 / pk["hbm_gbs"]})
        print(res[-1], flush=True)
        xr = x.detach().contiguous().requires_grad_()
        wr = w.clone().requires_grad_()
        y = ops.causal_conv1d(xr, wr, b, activation="silu", channel_last=True)
        g = torch.randn_like(y)
        t = time_ms(lambda: torch.autograd.grad(y, (xr, wr), g, retain_graph=True))
        res.append({"kernel": "causal_conv1d_bwd", "what": what, "shape": [B, L, Di], "ms": t, "gbs": 3 * x.numel() * 2 / t / 1e6})
        print(res[-1], flush=True)
        u = torch.randn(B, L, Di, device="cuda").bfloat16().requires_grad_()
        delta = (torch.randn(B, L, Di, device="cuda") * 0.5).bfloat16().requires_grad_()
        Bm = torch.randn(B, L, N, device="cuda").bfloat16().requires_grad_()
        Cm = torch.randn(B, L, N, device="cuda").bfloat16().requires_grad_()
        A = (-torch.exp(torch.rand(Di, N, device="cuda"))).requires_grad_()
        D, bias = torch.randn(Di, device="cuda").requires_grad_(), torch.randn(Di, device="cuda").requires_grad_()
        zz = z.detach().contiguous().requires_grad_()
        f = lambda: ops.selective_scan(u, delta, A, Bm, Cm, D, z=zz, delta_bias=bias, delta_softplus=True, channel_last=True)
        t_f = time_ms(f)
        y = f()
        g = torch.randn_like(y)
        t_b = time_ms(lambda: torch.autograd.grad(y, (u, delta, A, Bm, Cm, D, zz, bias), g, retain_graph=True), iters=5)
        by_f, by_b = 4 * u.numel() * 2, 8 * u.numel() * 2
        res.append({"kernel": "selective_scan", "what": what, "shape": [B, L, Di, N], "fwd_ms": t_f, "fwd_gbs": by_f / t_f / 1e6,
                    "bwd_ms": t_b, "bwd_gbs": by_b / t_b / 1e6, "steps_per_s": B * L * Di * N / t_f / 1e-3})
        print(res[-1], flush=True)


def bench_gdn(res: list) -> None:
    """Gated delta rule at the Gated-DeltaNet layer shape (6 heads, Dk 256, Dv 512): the recurrence kernel alone, and
    the whole op forward / forward+backward against the same chunk form with the recurrence as a PyTorch loop."""
    import importlib
    G = importlib.import_module("archscale_b200.ops.gated_delta_rule")
    ext = backend.require_extension()
    for (B, T, H, Dk, Dv) in [(1, 4096, 6, 256, 512), (8, 4096, 6, 256, 512)]:
        BH, nC = B * H, T // 64
        mk = lambda d, sc: (torch.randn(BH, T, d, device="cuda") * sc).bfloat16()
        a_op, bm_op, c_add, e_op, f_op = mk(Dk, 0.06), mk(Dk, 0.06), mk(Dv, 1.0), mk(Dv, 0.3), mk(Dk, 0.3)
        decay = torch.rand(BH, nC, device="cuda") * 0.5 + 0.5
        t_f = time_ms(lambda: ext.gdn_state(a_op, c_add, bm_op, None, None, decay, False, -1.0, 1.0))
        t_b = time_ms(lambda: ext.gdn_state(a_op, c_add, bm_op, e_op, f_op, decay, True, 1.0, -1.0))
        fl_f = 2.0 * BH * T * Dk * Dv * 2
        res.append({"kernel": "gdn_state", "shape": [B, T, H, Dk, Dv], "ctas": BH * Dv // 128, "fwd_pass_ms": t_f,
                    "fwd_tflops": fl_f / t_f / 1e9, "bwd_pass_ms": t_b, "bwd_tflops": 1.5 * fl_f / t_b / 1e9,
                    "us_per_chunk_fwd": t_f * 1e3 / nC / max(1, -(-BH * Dv // 128 // 148))})
        print(res[-1], flush=True)
        q, k = (torch.randn(B, T, H, Dk, device="cuda").bfloat16().requires_grad_() for _ in range(2))
        v = torch.randn(B, T, H, Dv, device="cuda").bfloat16().requires_grad_()
        g = (-torch.rand(B, T, H, device="cuda") * 0.3).requires_grad_()
        beta = (torch.rand(B, T, H, device="cuda") * 2).requires_grad_()
        row = {"kernel": "gated_delta_rule", "shape": [B, T, H, Dk, Dv]}
        for name, core in (("kernel", G._chunk_core), ("torch_loop", G._chunk_core_ref)):
            if name == "torch_loop" and B > 1:
                continue
            saved, G._chunk_core = G._chunk_core, core
            try:
                f = lambda: G.gated_delta_rule(q, k, v, g, beta)
                row[name + "_fwd_ms"] = time_ms(f, iters=3)

                def fb():
                    o = f()
                    torch.autograd.grad(o, (q, k, v, g, beta), torch.ones_like(o))
                row[name + "_fwd_bwd_ms"] = time_ms(fb, iters=3)
            finally:
                G._chunk_core = saved
        res.append(row)
        print(row, flush=True)


def bench_mxfp8(res: list) -> None:
    """Block-scaled MXFP8 GEMM and its quantisers against the bf16 tcgen05 kernel on the same shapes."""
    from archscale_b200.ops import mxfp8
    ext = backend.require_extension()
    pk = peaks()
    for (M, N, K, what) in [(32768, 3072, 2048, "fwd qkv d16"), (32768, 11264, 2048, "fwd w1 d16"),
                            (32768, 2048, 5632, "fwd w3 d16"), (8192, 8192, 8192, "square 8192")]:
        a, b = torch.randn(M, K, device="cuda").bfloat16(), torch.randn(N, K, device="cuda").bfloat16()
        aq, asf = mxfp8.quantize(a)
        bq, bsf = mxfp8.quantize(b)
        t_q = time_ms(lambda: mxfp8.gemm(aq, asf, bq, bsf))
        t_b = time_ms(lambda: ext.gemm_bf16(a, b, 0, torch.bfloat16, None))
        t_row = time_ms(lambda: mxfp8.quantize(a))
        t_col = time_ms(lambda: mxfp8.quantize(a, colwise=True))
        fl = 2.0 * M * N * K
        res.append({"kernel": "gemm_mxfp8", "case": what, "M": M, "N": N, "K": K, "ms": t_q, "tflops": fl / t_q / 1e9,
                    "bf16_kernel_ms": t_b, "speedup_vs_bf16_kernel": t_b / t_q,
                    "frac_of_" + pk["kind"] + "_bf16_peak": fl / t_q / 1e9 / pk["bf16_tflops"],
                    "quant_rowwise_ms": t_row, "quant_rowwise_gbs": 3.0 * M * K / t_row / 1e6,
                    "quant_colwise_ms": t_col, "quant_colwise_gbs": 3.0 * M * K / t_col / 1e6})
        print(res[-1], flush=True)


def bench_nvfp4(res: list) -> None:
    """NVFP4 block-scaled GEMM and its quantisers against the MXFP8 and bf16 tcgen05 kernels on the same shapes."""
    from archscale_b200.ops import mxfp8, nvfp4
    ext = backend.require_extension()
    pk = peaks()
    for (M, N, K, what) in [(32768, 3072, 2048, "fwd qkv d16"), (32768, 11264, 2048, "fwd w1 d16"),
                            (32768, 2048, 5632, "fwd w3 d16"), (8192, 8192, 8192, "square 8192")]:
        a, b = torch.randn(M, K, device="cuda").bfloat16(), torch.randn(N, K, device="cuda").bfloat16()
        qa, qb = nvfp4.quantize(a), nvfp4.quantize(b)
        ma, mb = mxfp8.quantize(a), mxfp8.quantize(b)
        t_q = time_ms(lambda: nvfp4.gemm(qa, qb))
        t_8 = time_ms(lambda: mxfp8.gemm(ma[0], ma[1], mb[0], mb[1]))
        t_b = time_ms(lambda: ext.gemm_bf16(a, b, 0, torch.bfloat16, None))
        am = nvfp4.amax(a)
        t_amax = time_ms(lambda: nvfp4.amax(a))
        t_row = time_ms(lambda: nvfp4.quantize(a, amax_t=am))
        t_both = time_ms(lambda: nvfp4.quantize_both(a, amax_t=am))
        fl = 2.0 * M * N * K
        res.append({"kernel": "gemm_nvfp4", "case": what, "M": M, "N": N, "K": K, "ms": t_q, "tflops": fl / t_q / 1e9,
                    "mxfp8_kernel_ms": t_8, "bf16_kernel_ms": t_b, "speedup_vs_bf16_kernel": t_b / t_q,
                    "frac_of_" + pk["kind"] + "_bf16_peak": fl / t_q / 1e9 / pk["bf16_tflops"],
                    "amax_ms": t_amax, "quant_rowwise_ms": t_row, "quant_both_orientations_ms": t_both})
        print(res[-1], flush=True)


ALL = {"gemm": bench_gemm, "rmsnorm": bench_rmsnorm, "swiglu": bench_swiglu, "ce": bench_ce, "rope": bench_rope,
       "attn": bench_attn, "mamba": bench_mamba, "mxfp8": bench_mxfp8, "nvfp4": bench_nvfp4, "gdn": bench_gdn}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("which", nargs="*", default=list(ALL))
    ap.add_argument("--json", default=None)
    a = ap.parse_args()
    torch.set_float32_matmul_precision("high")          # as the trainer sets it: fp32 matmuls of the chunked scans on TF32
    res: list = []
    for w in a.which:
        ALL[w](res)
    status = backend.require_extension().device_status()
    print("device status word:", status)
    if a.json:
        json.dump({"peaks": peaks(), "results": res, "device_status": status}, open(a.json, "w"), indent=1)


if __name__ == "__main__":
    main()
