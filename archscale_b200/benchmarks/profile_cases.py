"""One kernel, one small case, three launches: the program to put under ``ncu``.

Inputs are larger than the 126 MB L2 (so DRAM counters mean something) and well under a few GB; there is
no warm-up loop and no timing, so a capture with ``-k regex:<kernel> -c 3`` ends by itself quickly.

    python -m archscale_b200.benchmarks.profile_cases gemm
    ncu --set full --clock-control none -k regex:gemm2_bf16_kernel -c 3 -o prof python -m archscale_b200.benchmarks.profile_cases gemm
"""
from __future__ import annotations

import sys

import torch

from archscale_b200 import ops
from archscale_b200.ops import backend


def _run(fn, n: int = 3) -> None:
    for _ in range(n):
        fn()
    torch.cuda.synchronize()


def case_gemm():
    ext = backend.require_extension()
    a, b = torch.randn(8192, 4096, device="cuda").bfloat16(), torch.randn(8192, 4096, device="cuda").bfloat16()
    _run(lambda: ext.gemm_bf16(a, b, 0, torch.bfloat16, None))


def case_gemm_wgrad():
    ext = backend.require_extension()
    a, b = torch.randn(16384, 4096, device="cuda").bfloat16(), torch.randn(16384, 4096, device="cuda").bfloat16()
    acc = torch.zeros(4096, 4096, device="cuda")
    _run(lambda: ext.gemm_bf16(a, b, 2, torch.float32, acc))


def case_mxfp8():
    from archscale_b200.ops import mxfp8
    a, b = torch.randn(8192, 4096, device="cuda").bfloat16(), torch.randn(8192, 4096, device="cuda").bfloat16()
    aq, asf = mxfp8.quantize(a)
    bq, bsf = mxfp8.quantize(b)
    mxfp8.quantize(a, colwise=True)
    _run(lambda: mxfp8.gemm(aq, asf, bq, bsf))


def case_nvfp4():
    from archscale_b200.ops import nvfp4
    a, b = torch.randn(8192, 4096, device="cuda").bfloat16(), torch.randn(8192, 4096, device="cuda").bfloat16()
    qa, qb = nvfp4.quantize(a), nvfp4.quantize(b)
    _run(lambda: nvfp4.gemm(qa, qb))


def _qkv(B=4, T=4096, H=16, G=4, D=128):
    mk = lambda h: torch.randn(B, T, h, D, device="cuda").bfloat16().requires_grad_()
    return mk(H), mk(G), mk(G)


def case_attn_fwd():
    q, k, v = _qkv()
    with torch.no_grad():
        _run(lambda: ops.attention(q, k, v))


def case_attn_bwd():
    q, k, v = _qkv()
    o = ops.attention(q, k, v)
    g = torch.randn_like(o)
    _run(lambda: torch.autograd.grad(o, (q, k, v), g, retain_graph=True))


def case_rmsnorm():
    x = torch.randn(65536, 2048, device="cuda").bfloat16().requires_grad_()
    w = torch.ones(2048, device="cuda").bfloat16().requires_grad_()
    y = ops.rms_norm(x, w, 1e-5)
    g = torch.randn_like(y)
    _run(lambda: torch.autograd.grad(ops.rms_norm(x, w, 1e-5), (x, w), g))


def case_swiglu():
    g, u = torch.randn(65536, 5632, device="cuda").bfloat16().requires_grad_(), torch.randn(65536, 5632, device="cuda").bfloat16()
    dy = torch.randn_like(u)
    _run(lambda: torch.autograd.grad(ops.swiglu(g, u), g, dy))


def case_ce():
    from archscale_b200.ops.cross_entropy import FusedLinearCrossEntropyLoss
    tgt = torch.randint(0, 32000, (8192,), device="cuda")
    h = torch.randn(8192, 2048, device="cuda").bfloat16().requires_grad_()
    w = (torch.randn(32000, 2048, device="cuda") * 0.02).bfloat16().requires_grad_()
    _run(lambda: FusedLinearCrossEntropyLoss()(h, w, tgt).backward())


def case_scan():
    B, L, Di, N = 2, 4096, 4096, 16
    mk = lambda *s: torch.randn(*s, device="cuda").bfloat16().requires_grad_()
    u, delta, z, Bm, Cm = mk(B, L, Di), mk(B, L, Di), mk(B, L, Di), mk(B, L, N), mk(B, L, N)
    A = (-torch.exp(torch.rand(Di, N, device="cuda"))).requires_grad_()
    D, bias = torch.randn(Di, device="cuda").requires_grad_(), torch.randn(Di, device="cuda").requires_grad_()

    def once():
        y = ops.selective_scan(u, delta, A, Bm, Cm, D, z=z, delta_bias=bias, delta_softplus=True, channel_last=True)
        torch.autograd.grad(y, (u, delta, A, Bm, Cm, D, z, bias), torch.ones_like(y))
    _run(once)


def case_conv1d():
    x = torch.randn(8, 4096, 4096, device="cuda").bfloat16().requires_grad_()
    w, b = torch.randn(4096, 4, device="cuda").requires_grad_(), torch.randn(4096, device="cuda").requires_grad_()

    def once():
        y = ops.causal_conv1d(x, w, b, activation="silu", channel_last=True)
        torch.autograd.grad(y, (x, w, b), torch.ones_like(y))
    _run(once)


def case_moe():
    from archscale_b200.ops.grouped_gemm import moe_ffn_cuda
    T, C, E, K, I = 16384, 1024, 64, 8, 256
    x = torch.randn(T, C, device="cuda").bfloat16().requires_grad_()
    w1 = (torch.randn(E, 2 * I, C, device="cuda") * 0.02).bfloat16().requires_grad_()
    w2 = (torch.randn(E, C, I, device="cuda") * 0.02).bfloat16().requires_grad_()
    logits = torch.randn(T, E, device="cuda")
    scores, idx = torch.topk(torch.softmax(logits, -1), K)

    def once():
        y = moe_ffn_cuda(x, w1, w2, scores.to(torch.float32), idx)
        y.float().sum().backward()
    _run(once)


def case_gdn():
    """One forward pass and one reversed pass (with the extra term) of the gated-delta-rule recurrence kernel."""
    ext = backend.require_extension()
    BH, T, Dk, Dv = 12, 4096, 256, 512
    mk = lambda d, sc: (torch.randn(BH, T, d, device="cuda") * sc).bfloat16()
    a_op, bm_op, c_add, e_op, f_op = mk(Dk, 0.06), mk(Dk, 0.06), mk(Dv, 1.0), mk(Dv, 0.3), mk(Dk, 0.3)
    decay = torch.rand(BH, T // 64, device="cuda") * 0.5 + 0.5
    ext.gdn_state(a_op, c_add, bm_op, None, None, decay, False, -1.0, 1.0)
    ext.gdn_state(a_op, c_add, bm_op, e_op, f_op, decay, True, 1.0, -1.0)
    torch.cuda.synchronize()


CASES = {k[5:]: v for k, v in list(globals().items()) if k.startswith("case_")}


def main() -> None:
    name = sys.argv[1] if len(sys.argv) > 1 else "gemm"
    CASES[name]()
    print(name, "done; device status", backend.require_extension().device_status())


if __name__ == "__main__":
    main()
