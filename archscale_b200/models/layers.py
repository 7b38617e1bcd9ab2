"""``Linear``: an ``nn.Linear`` whose matmuls run the tcgen05 GEMM (or its MXFP8 variant)."""
from __future__ import annotations

import torch
import torch.nn as nn

from archscale_b200 import ops


class Linear(nn.Linear):
    """Drop-in ``nn.Linear`` (same parameter names / state-dict keys).

    * bf16 CUDA inputs → ``ops.linear`` (hand-written GEMM for fwd, dgrad, wgrad);
    * ``mxfp8=True`` → block-scaled E4M3 GEMM with bf16 master weights
      (replaces the ``te.Linear`` swap of the reference, `precision.py:192-251`);
    * ``nvfp4=True`` → NVFP4 GEMM (e2m1 elements, E4M3 block scales; the ``--fp4`` recipe, `precision.py:92-96`),
      emulated in PyTorch off the GPU;
    * anything else (CPU, fp32) → ``F.linear``.
    The weight is cast to the activation dtype when they differ (fp32 masters, bf16 compute).
    """

    mxfp8: bool = False
    nvfp4: bool = False

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        w, b = self.weight, self.bias
        g = getattr(w, "_fsdp_group", None)
        if g is not None and getattr(g, "ag_pending", False) and (self.mxfp8 or self.nvfp4 or not (
                w._fsdp_first and x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16)):
            w._fsdp_engine.finish_pending_gather(g)
        if w.dtype != x.dtype:
            w = w.to(x.dtype)
            b = b.to(x.dtype) if b is not None else None
        if self.nvfp4:
            from archscale_b200.ops import nvfp4
            return nvfp4.linear_nvfp4(x, w, b)
        if self.mxfp8 and x.is_cuda:
            from archscale_b200.ops import mxfp8
            return mxfp8.linear_mxfp8(x, w, b)
        return ops.linear(x, w, b)


def apply_mxfp8(model: nn.Module, skip=("lm_head", "lc_proj")) -> int:
    """Switch every :class:`Linear` of ``model`` to the MXFP8 path, except modules whose name contains one of
    ``skip`` and layers whose dimensions are not multiples of 128 (the rule of `precision.py:192-251`, with
    the block-scaled kernel's granularity instead of 16).  Returns the number of layers switched."""
    n = 0
    for name, mod in model.named_modules():
        if isinstance(mod, Linear) and not any(s in name for s in skip) \
                and mod.in_features % 128 == 0 and mod.out_features % 128 == 0:
            mod.mxfp8 = True
            n += 1
    return n


def apply_nvfp4(model: nn.Module, skip=("lm_head", "lc_proj")) -> int:
    """Switch every :class:`Linear` of ``model`` to the NVFP4 path, with the same exclusions as :func:`apply_mxfp8` and
    the NVFP4 kernels' granularity (multiples of 256).  Returns the number of layers switched."""
    n = 0
    for name, mod in model.named_modules():
        if isinstance(mod, Linear) and not any(s in name for s in skip) \
                and mod.in_features % 256 == 0 and mod.out_features % 256 == 0:
            mod.nvfp4 = True
            n += 1
    return n
