"""Guarded allocations and run-twice comparisons for kernel tests.

No memory checker runs on the target GPUs, so out-of-bounds writes and races are looked for the slow way:

* :func:`guarded` returns a tensor that sits between two guard bands filled with a bit pattern; :func:`guards_intact` tells after
  a kernel ran whether anything wrote outside the tensor (a write past either end of an output or an in-place operand);
* :func:`bitwise_repeatable` runs a function twice on the same inputs and compares every output bit for bit — a data race between
  CTAs, an atomic whose order matters or an uninitialised read shows up as a difference.
"""
from __future__ import annotations

from typing import Callable, Sequence, Tuple

import torch

_GUARD_BYTES = 4096
_PATTERN = 0xA5


def guarded(shape: Sequence[int], dtype: torch.dtype, device, fill: float = 0.0) -> Tuple[torch.Tensor, torch.Tensor]:
    """(tensor view of ``shape``, the whole byte buffer).  The view is contiguous, 256-byte aligned and has ``_GUARD_BYTES`` of
    pattern on both sides."""
    numel = 1
    for s in shape:
        numel *= int(s)
    nbytes = numel * torch.empty(0, dtype=dtype).element_size()
    body = (nbytes + 255) // 256 * 256
    raw = torch.full((2 * _GUARD_BYTES + body,), _PATTERN, dtype=torch.uint8, device=device)
    view = raw[_GUARD_BYTES:_GUARD_BYTES + nbytes].view(dtype).view(*shape)
    view.fill_(fill)
    return view, raw


def guards_intact(view: torch.Tensor, raw: torch.Tensor) -> bool:
    nbytes = view.numel() * view.element_size()
    lo = raw[:_GUARD_BYTES]
    hi = raw[_GUARD_BYTES + nbytes:]
    return bool((lo == _PATTERN).all()) and bool((hi == _PATTERN).all())


def bitwise_repeatable(fn: Callable[[], object]) -> bool:
    """True when two calls of ``fn`` return bitwise equal tensors (a tensor or a tuple / list of tensors; None entries skipped)."""
    def flat(o):
        if o is None:
            return []
        if isinstance(o, torch.Tensor):
            return [o]
        out = []
        for x in o:
            out += flat(x)
        return out
    a = [t.detach().clone() for t in flat(fn())]
    b = flat(fn())
    if len(a) != len(b):
        return False
    return all(x.shape == y.shape and torch.equal(x.view(torch.uint8) if x.dtype != torch.bool else x,
                                                  y.view(torch.uint8) if y.dtype != torch.bool else y) for x, y in zip(a, b))
