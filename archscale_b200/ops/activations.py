"""SwiGLU / GLU / GPT-OSS SwiGLU / relu² elementwise ops.

Behavioural reference: `lit_gpt/gated_memory_unit.py:14-74` (``swiglu(x, y) = x·σ(x)·y``,
``glu(x, y) = σ(x)·y`` with fp32 internals) and `lit_gpt/model.py:608-618` (GPT-OSS variant).

CUDA path: ``csrc/elementwise.cu`` — 16-byte vector loads, fp32 math; the packed variant
reads the ``[gate | up]`` halves of a GEMM output in place (no ``chunk`` copies).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from . import backend


def swiglu_ref(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    return (F.silu(gate.float()) * up.float()).to(gate.dtype)


def glu_ref(g: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
    return (torch.sigmoid(g.float()) * y.float()).to(y.dtype)


def oss_swiglu_ref(x_glu: torch.Tensor, x_lin: torch.Tensor, alpha: float = 1.702, limit: float = 7.0):
    x_glu = x_glu.clamp(max=limit)
    x_lin = x_lin.clamp(min=-limit, max=limit)
    return x_glu * torch.sigmoid(alpha * x_glu) * (x_lin + 1)


class _SwiGLUPackedFn(torch.autograd.Function):
    """y = silu(x[:, :I]) * x[:, I:] for a packed (N, 2I) bf16 activation."""

    @staticmethod
    def forward(ctx, x):
        ext = backend.require_extension()
        ctx.save_for_backward(x)
        backend.count_launch()
        return ext.swiglu_packed_fwd(x)

    @staticmethod
    def backward(ctx, dy):
        ext = backend.require_extension()
        (x,) = ctx.saved_tensors
        backend.count_launch()
        return ext.swiglu_packed_bwd(x, dy.contiguous())


class _SwiGLUFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gate, up):
        ext = backend.require_extension()
        gate, up = gate.contiguous(), up.contiguous()
        ctx.save_for_backward(gate, up)
        backend.count_launch()
        return ext.swiglu_fwd(gate, up)

    @staticmethod
    def backward(ctx, dy):
        ext = backend.require_extension()
        gate, up = ctx.saved_tensors
        backend.count_launch()
        dg, du = ext.swiglu_bwd(gate, up, dy.contiguous())
        return dg, du


def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    if (gate.dtype == torch.bfloat16 and up.dtype == torch.bfloat16 and gate.shape == up.shape
            and gate.numel() % 8 == 0 and backend.use_cuda_kernel("swiglu", gate, up)):
        return _SwiGLUFn.apply(gate, up)
    return swiglu_ref(gate, up)


def swiglu_packed(x: torch.Tensor) -> torch.Tensor:
    """SwiGLU over the two halves of the last dim: ``silu(x[..., :I]) * x[..., I:]``."""
    I = x.shape[-1] // 2
    if (x.dtype == torch.bfloat16 and I % 8 == 0 and x.is_contiguous()
            and backend.use_cuda_kernel("swiglu", x)):
        return _SwiGLUPackedFn.apply(x.view(-1, 2 * I)).view(*x.shape[:-1], I)
    g, u = x.chunk(2, dim=-1)
    return swiglu_ref(g, u)


def glu(g: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
    return glu_ref(g, y)
