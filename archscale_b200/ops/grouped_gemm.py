"""Grouped expert GEMMs on the tcgen05 path (python side).

See :mod:`archscale_b200.ops.moe` for semantics.  The kernels take *device-side* expert
offsets, so no token count ever travels to the host (the reference syncs per layer,
`lit_gpt/moe.py:622-623`).
"""
from __future__ import annotations

import torch

from . import backend


def supported(x, w_in, w_out, b_in, b_out) -> bool:
    if not x.is_cuda or b_in is not None or b_out is not None:
        return False
    ext = backend.load_extension()
    if ext is None or not hasattr(ext, "grouped_gemm_bf16"):
        return False
    C = x.shape[1]
    I2 = w_in.shape[1]
    return (x.dtype == torch.bfloat16 and w_in.dtype == torch.bfloat16 and w_out.dtype == torch.bfloat16
            and C % 64 == 0 and I2 % 128 == 0)


def moe_ffn_cuda(x, w_in, w_out, scores, indices):
    raise NotImplementedError
