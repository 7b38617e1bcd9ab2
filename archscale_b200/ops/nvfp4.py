"""NVFP4 linear layers: e2m1 elements, one unsigned E4M3 scale per 16 elements along the contraction dimension and one
fp32 scale per tensor (``x ≈ tensor_scale · block_scale · e2m1``).

Replaces the ``te.Linear`` + ``NVFP4BlockScaling`` recipe the reference selects with ``--fp4``
(`precision.py:92-96`, `pretrain.py:250,411`).  The master weight stays bf16/fp32; every GEMM of the layer quantises its
operands on the fly, with the same three K-major "NT" products as :mod:`archscale_b200.ops.mxfp8`:

* forward  ``y  = Q_row(x)  · Q_row(W)ᵀ``
* dgrad    ``dx = Q_row(dy) · Q_col(W)ᵀ``
* wgrad    ``dW = Q_col(dy) · Q_col(x)ᵀ``, accumulated into fp32 ``main_grad`` when the engine provides one

Two implementations of the same arithmetic:

* the kernel path (``csrc/gemm_mxfp8.cu``: ``tcgen05.mma.kind::mxf4nvf4.block_scale.scale_vec::4X`` and the quantisers),
  scales along one dimension for weights as for activations;
* the emulated path (plain PyTorch, any device): quantise → dequantise → matmul.  It is the CPU path and the test oracle
  (``ARCHSCALE_B200_NVFP4=emulate`` selects it on a GPU).

Both apply the two gradient-side options of the recipe by default: stochastic rounding of the gradient operands (round to
nearest everywhere else) and a random 16 × 16 Hadamard transform of both weight-gradient operands along the token dimension
(``ARCHSCALE_B200_NVFP4_SR=0`` / ``ARCHSCALE_B200_NVFP4_RHT=0`` switch them off).  The kernels draw their random numbers from a
counter hash and scale a transformed operand from 4 · amax (the bound of a transformed element), so the two paths agree in
distribution, not bit for bit, once an option is on.

Quantisation rule (both paths, bit for bit): ``tensor_scale = amax(x) / (6·448)`` (1 for an all-zero tensor);
``block_scale = E4M3(amax_block · (1 / (6 · tensor_scale)))`` rounded to nearest (each step in fp32);
``element = e2m1(x · (1 / (block_scale · tensor_scale)))`` rounded to nearest even and saturated at ±6.
"""
from __future__ import annotations

import os
from typing import Optional, Tuple

import torch

from . import backend

E2M1_MAX = 6.0
E4M3_MAX = 448.0
_GRID = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)


def _grid(device) -> torch.Tensor:
    return torch.tensor(_GRID, dtype=torch.float32, device=device)


# ------------------------------------------------------------------------------------------------ references
def tensor_amax(x: torch.Tensor) -> torch.Tensor:
    """fp32 [1]: the largest magnitude of the tensor (one pass, no host synchronisation)."""
    return torch.linalg.vector_norm(x.detach().reshape(-1), float("inf")).float().reshape(1)


def scale_from_amax(amax: torch.Tensor) -> torch.Tensor:
    """``amax · (1 / (6·448))`` in fp32, or 1 when the tensor is all zero: the rule the kernels apply to the same number."""
    return torch.where(amax > 0, amax * (1.0 / (E2M1_MAX * E4M3_MAX)), torch.ones_like(amax))


def tensor_scale(x: torch.Tensor) -> torch.Tensor:
    return scale_from_amax(tensor_amax(x))


def _codes_nearest(a: torch.Tensor) -> torch.Tensor:
    """|value| → e2m1 magnitude code 0..7, round to nearest, ties to the even code."""
    return ((a > 0.25).to(torch.uint8) + (a >= 0.75).to(torch.uint8) + (a > 1.25).to(torch.uint8) + (a >= 1.75).to(torch.uint8)
            + (a > 2.5).to(torch.uint8) + (a >= 3.5).to(torch.uint8) + (a > 5.0).to(torch.uint8))


def _codes_stochastic(a: torch.Tensor, generator: Optional[torch.Generator]) -> torch.Tensor:
    """|value| → code, rounding up with probability (a − lower) / (upper − lower)."""
    g = _grid(a.device)
    lo = (torch.bucketize(a, g, right=True) - 1).clamp(0, 7)
    hi = (lo + 1).clamp(max=7)
    glo, ghi = g[lo], g[hi]
    p = torch.where(ghi > glo, (a - glo) / (ghi - glo).clamp_min(1e-30), torch.zeros_like(a))
    u = torch.rand(a.shape, device=a.device, generator=generator)
    return torch.where(u < p, hi, lo).to(torch.uint8)


def quantize_ref(x: torch.Tensor, ts: Optional[torch.Tensor] = None, stochastic: bool = False,
                 generator: Optional[torch.Generator] = None) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Row-wise NVFP4 of x:(R,K), K % 16 == 0 → (packed uint8 (R,K/2), E4M3 scale bits uint8 (R,K/16), tensor scale fp32 [1])."""
    R, K = x.shape
    if ts is None:
        ts = tensor_scale(x)
    xb = x.float().view(R, K // 16, 16)
    amax = xb.abs().amax(-1)
    sb8 = (amax * torch.reciprocal(ts * E2M1_MAX)).clamp(max=E4M3_MAX).to(torch.float8_e4m3fn)
    sb = sb8.float()
    inv = torch.where(sb > 0, torch.reciprocal(sb * ts), torch.zeros_like(sb))
    a = xb.abs() * inv.unsqueeze(-1)
    code = _codes_stochastic(a, generator) if stochastic else _codes_nearest(a)
    code = code | ((xb * inv.unsqueeze(-1)) < 0).to(torch.uint8) * 8
    code = code.view(R, K)
    packed = code[:, 0::2] | (code[:, 1::2] << 4)
    return packed.contiguous(), sb8.view(torch.uint8), ts


def dequantize_ref(packed: torch.Tensor, sb_bits: torch.Tensor, ts: torch.Tensor) -> torch.Tensor:
    R, K2 = packed.shape
    K = 2 * K2
    code = torch.stack((packed & 0xF, packed >> 4), dim=-1).view(R, K).long()
    mag = _grid(packed.device)[code & 7]
    val = torch.where((code & 8) != 0, -mag, mag)
    sb = sb_bits.view(torch.float8_e4m3fn).float()
    return (val.view(R, K // 16, 16) * (sb * ts).unsqueeze(-1)).view(R, K)


def fake_quantize(x: torch.Tensor, stochastic: bool = False, generator: Optional[torch.Generator] = None) -> torch.Tensor:
    """Round x:(R,K) to its NVFP4 representation along K and return it in fp32."""
    return dequantize_ref(*quantize_ref(x, None, stochastic, generator))


def hadamard16(device, dtype=torch.float32) -> torch.Tensor:
    """Orthonormal 16 × 16 Sylvester Hadamard matrix."""
    h = torch.ones(1, 1, device=device, dtype=dtype)
    for _ in range(4):
        h = torch.cat((torch.cat((h, h), 1), torch.cat((h, -h), 1)), 0)
    return h / 4.0


def random_hadamard(x: torch.Tensor, sign: torch.Tensor) -> torch.Tensor:
    """x:(R,K) → x · blockdiag(diag(sign) · H16) along K.  Orthogonal, so products over K are unchanged."""
    R, K = x.shape
    m = sign.to(x.dtype).unsqueeze(1) * hadamard16(x.device, x.dtype)
    return (x.view(R, K // 16, 16) @ m).view(R, K)


_RHT_SIGN = None


def _rht_sign(device) -> torch.Tensor:
    """One fixed ±1 vector for the whole run (the recipe draws it once)."""
    global _RHT_SIGN
    if _RHT_SIGN is None:
        g = torch.Generator().manual_seed(0x5EED)
        _RHT_SIGN = (torch.randint(0, 2, (16,), generator=g) * 2 - 1).float()
    return _RHT_SIGN.to(device)


def _opt(name: str, default: str = "1") -> bool:
    return os.environ.get(name, default) != "0"


class _LinearNVFP4EmulatedFn(torch.autograd.Function):
    """The three products on fake-quantised operands (fp32 matmuls); any device."""

    @staticmethod
    def forward(ctx, x, weight, bias, stochastic, rht):
        x2 = x.reshape(-1, x.shape[-1])
        y = (fake_quantize(x2) @ fake_quantize(weight).t()).to(x.dtype)
        if bias is not None:
            y = y + bias.to(y.dtype)
        ctx.save_for_backward(x2, weight)
        ctx.opts = (bias is not None, x.shape, bool(stochastic), bool(rht))
        ctx.weight_ref = weight
        return y.view(*x.shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, weight = ctx.saved_tensors
        has_bias, x_shape, stochastic, rht = ctx.opts
        dy2 = dy.reshape(-1, dy.shape[-1])
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            wt = fake_quantize(weight.t().contiguous())                 # (K, N): blocks along out_features
            dx = (fake_quantize(dy2, stochastic) @ wt.t()).to(dy.dtype).view(x_shape)
        if ctx.needs_input_grad[1]:
            gt, xt = dy2.t().contiguous().float(), x2.t().contiguous().float()      # (N, T), (K, T): blocks along tokens
            if rht:
                s = _rht_sign(dy.device)
                gt, xt = random_hadamard(gt, s), random_hadamard(xt, s)
            prod = fake_quantize(gt, stochastic) @ fake_quantize(xt).t()
            main_grad = getattr(ctx.weight_ref, "main_grad", None)
            if main_grad is not None:
                main_grad.add_(prod)
            else:
                dw = prod.to(weight.dtype)
        if has_bias and ctx.needs_input_grad[2]:
            db = dy2.float().sum(0).to(dy.dtype)
        return dx, dw, db, None, None


def emulated_supported(x2: torch.Tensor, weight: torch.Tensor) -> bool:
    return x2.shape[1] % 16 == 0 and weight.shape[0] % 16 == 0 and x2.shape[0] % 16 == 0


def linear_nvfp4_emulated(x, weight, bias=None, stochastic: Optional[bool] = None, rht: Optional[bool] = None):
    stochastic = _opt("ARCHSCALE_B200_NVFP4_SR") if stochastic is None else stochastic
    rht = _opt("ARCHSCALE_B200_NVFP4_RHT") if rht is None else rht
    return _LinearNVFP4EmulatedFn.apply(x, weight, bias, stochastic, rht)


# ------------------------------------------------------------------------------------------------ kernels
# A quantised operand is a triple (packed e2m1 bytes, chunked E4M3 block scales, fp32 [1] largest magnitude of the source
# tensor); the kernels derive the tensor scale from the last item themselves.
def amax(x: torch.Tensor) -> torch.Tensor:
    ext = backend.require_extension()
    backend.count_launch()
    return ext.nvfp4_amax(x)


_SEED = [0x1234567]


def _next_seed() -> int:
    """A new 31-bit seed per stochastic quantisation (a counter through an odd multiplier: no two calls of a run share numbers)."""
    _SEED[0] = (_SEED[0] * 1103515245 + 12345) & 0x7FFFFFFF
    return _SEED[0]


def _sign_mask() -> int:
    """The fixed ±1 vector of the Hadamard transform as a bit mask (bit j set: element j is negated)."""
    sign = _rht_sign("cpu")
    return int(sum(1 << j for j in range(16) if sign[j] < 0))


def quantize(x: torch.Tensor, colwise: bool = False, amax_t: Optional[torch.Tensor] = None, stochastic: bool = False,
             rht: bool = False):
    """x:(R,C) bf16 → operand triple.  ``colwise`` returns the transposed operand (C,R/2); ``rht`` (transposed operand only)
    applies the random Hadamard transform to its 16-element blocks, ``stochastic`` rounds the elements stochastically."""
    ext = backend.require_extension()
    if amax_t is None:
        amax_t = amax(x)
    rht = rht and colwise
    backend.count_launch()
    q, sf = ext.nvfp4_quantize(x, amax_t, 1 if colwise else 0, stochastic, _next_seed() if stochastic else 0, rht,
                               _sign_mask() if rht else 0)
    return q, sf, (amax_t * 4.0 if rht else amax_t)


def quantize_both(x: torch.Tensor, amax_t: Optional[torch.Tensor] = None, stochastic: bool = False, rht: bool = False):
    """x:(R,C) bf16 → (row-wise operand, transposed operand) from one read of x; ``rht`` transforms the transposed one."""
    ext = backend.require_extension()
    if amax_t is None:
        amax_t = amax(x)
    backend.count_launch()
    q, sf, qt, sft = ext.nvfp4_quantize(x, amax_t, 2, stochastic, _next_seed() if stochastic else 0, rht,
                                        _sign_mask() if rht else 0)
    return (q, sf, amax_t), (qt, sft, amax_t * 4.0 if rht else amax_t)


def gemm(a, b, out_f32: bool = False, acc: Optional[torch.Tensor] = None, alpha: float = 1.0):
    """``a · bᵀ`` for two operand triples → (M,N) bf16 / fp32, or ``acc += …`` (fp32)."""
    ext = backend.require_extension()
    backend.count_launch()
    return ext.gemm_nvfp4(a[0], a[1], a[2], b[0], b[1], b[2], out_f32, acc, alpha)


def supported(x2: torch.Tensor, weight: torch.Tensor) -> bool:
    """Shapes the NVFP4 kernels take: every contraction dimension a multiple of 256."""
    T, K = x2.shape
    N = weight.shape[0]
    return (x2.is_cuda and x2.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and K % 256 == 0 and N % 256 == 0
            and T % 256 == 0 and backend.has("gemm_nvfp4"))


# quantised weights are reused until the weights change, like the MXFP8 ones (see ops/mxfp8.py)
_W_EPOCH = 0
_W_CACHE: dict = {}


def invalidate_weight_cache() -> None:
    global _W_EPOCH
    _W_EPOCH += 1
    _W_CACHE.clear()


def quantize_weight(weight: torch.Tensor, colwise: bool):
    key = (id(weight), colwise)
    tag = (_W_EPOCH, weight.data_ptr(), weight._version, tuple(weight.shape))
    hit = _W_CACHE.get(key)
    if hit is not None and hit[0] == tag:
        return hit[1]
    out = quantize(weight, colwise)
    _W_CACHE[key] = (tag, out)
    return out


class _LinearNVFP4Fn(torch.autograd.Function):
    """Each tensor is read twice per use at most: once for its largest magnitude, once by a quantiser that writes every
    orientation the step needs (x: row-wise for the forward product and transposed for the weight gradient, saved in place
    of x itself; dy: row-wise for dgrad and transposed for wgrad).  ``stochastic``: the gradient operands are rounded
    stochastically; ``rht``: both operands of the weight-gradient product get the random Hadamard transform."""

    @staticmethod
    def forward(ctx, x, weight, bias, stochastic, rht):
        x2 = x.reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        if ctx.needs_input_grad[1]:
            xq, xt = quantize_both(x2, rht=rht)
            ctx.save_for_backward(weight, *xt)
        else:
            xq = quantize(x2)
            ctx.save_for_backward(weight)
        y = gemm(xq, quantize_weight(weight, False))
        if bias is not None:
            y = y + bias.to(y.dtype)
        ctx.has_bias = bias is not None
        ctx.weight_ref = weight
        ctx.x_shape = x.shape
        ctx.opts = (bool(stochastic), bool(rht))
        return y.view(*x.shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, dy):
        weight, *xt = ctx.saved_tensors
        stochastic, rht = ctx.opts
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = dw = db = None
        need_dx, need_dw = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        if need_dx and need_dw:
            g, gt = quantize_both(dy2, stochastic=stochastic, rht=rht)
        elif need_dx:
            g, gt = quantize(dy2, stochastic=stochastic), None
        else:
            g, gt = None, quantize(dy2, colwise=True, stochastic=stochastic, rht=rht)
        if need_dx:
            dx = gemm(g, quantize_weight(weight, True)).view(ctx.x_shape)       # Wᵀ: (K, N) blocks along N
        if need_dw:
            main_grad = getattr(ctx.weight_ref, "main_grad", None)
            if main_grad is not None:
                gemm(gt, tuple(xt), acc=main_grad)                              # dyᵀ · (xᵀ)ᵀ, blocks along the tokens
            else:
                dw = gemm(gt, tuple(xt)).to(weight.dtype)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy2.float().sum(0).to(dy.dtype)
        return dx, dw, db, None, None


def linear_nvfp4(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """NVFP4 ``x @ weightᵀ + bias``.  CUDA bf16 tensors of supported shapes run the tcgen05 kernels; other tensors whose
    dimensions are multiples of 16 run the emulated path; the rest run an ordinary linear."""
    x2 = x.reshape(-1, x.shape[-1])
    mode = os.environ.get("ARCHSCALE_B200_NVFP4", "kernel")
    if mode != "emulate" and supported(x2, weight) and backend.use_cuda_kernel("nvfp4", x2, weight):
        return _LinearNVFP4Fn.apply(x, weight, bias, _opt("ARCHSCALE_B200_NVFP4_SR"), _opt("ARCHSCALE_B200_NVFP4_RHT"))
    if emulated_supported(x2, weight):
        return linear_nvfp4_emulated(x, weight, bias)
    from .gemm import linear
    return linear(x, weight, bias)
