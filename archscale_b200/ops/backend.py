"""Loader for the in-tree sm_100a extension and the policy for choosing a kernel.

Every op in :mod:`archscale_b200.ops` has two implementations:

* a plain PyTorch one (``*_ref``), which is the CPU backend and the numerical oracle, and
* a hand-written sm_100a CUDA kernel in ``archscale_b200/_C*.so``.

CUDA tensors take the kernel path.  If the extension cannot be loaded on a machine that
has a GPU, ops raise instead of silently running the PyTorch path, unless
``ARCHSCALE_B200_ALLOW_FALLBACK=1`` is set (used only to bisect a numerical problem).
``ARCHSCALE_B200_DISABLE=op1,op2`` forces the listed ops onto the PyTorch path.
"""
from __future__ import annotations

import glob
import importlib.util
import os
import threading
from typing import Optional

import torch

_lock = threading.Lock()
_ext = None
_ext_error: Optional[BaseException] = None
_launch_count = 0  # kernels of this package launched (maintained by the op wrappers)


def _pkg_dir() -> str:
    return os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def extension_path() -> Optional[str]:
    hits = sorted(glob.glob(os.path.join(_pkg_dir(), "_C*.so")))
    return hits[0] if hits else None


def load_extension():
    """Import ``archscale_b200._C`` (built by :mod:`archscale_b200.build`); cache the result."""
    global _ext, _ext_error
    if _ext is not None or _ext_error is not None:
        return _ext
    with _lock:
        if _ext is not None or _ext_error is not None:
            return _ext
        path = extension_path()
        if path is None:
            _ext_error = FileNotFoundError(
                "archscale_b200/_C*.so not found; run `python -m archscale_b200.build`")
            return None
        try:
            spec = importlib.util.spec_from_file_location("archscale_b200._C", path)
            mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(mod)
            _ext = mod
        except BaseException as e:  # noqa: BLE001 - surfaced by require_extension()
            _ext_error = e
    return _ext


def require_extension():
    ext = load_extension()
    if ext is None:
        raise RuntimeError(f"sm_100a extension unavailable: {_ext_error!r}")
    return ext


def _disabled(op: str) -> bool:
    v = os.environ.get("ARCHSCALE_B200_DISABLE", "")
    return bool(v) and (v == "all" or op in v.split(","))


def use_cuda_kernel(op: str, *tensors: torch.Tensor) -> bool:
    """True when ``op`` must run its sm_100a kernel for these tensors."""
    if not tensors or not all(t is None or t.is_cuda for t in tensors):
        return False
    if _disabled(op):
        return False
    if load_extension() is None:
        if os.environ.get("ARCHSCALE_B200_ALLOW_FALLBACK", "0") == "1":
            return False
        raise RuntimeError(
            f"op '{op}' got CUDA tensors but the sm_100a extension is not loadable: {_ext_error!r}. "
            "Build it with `python -m archscale_b200.build` (or set ARCHSCALE_B200_ALLOW_FALLBACK=1).")
    return True


def has(symbol: str) -> bool:
    """True when the loaded extension exports ``symbol`` (kernels land one by one)."""
    ext = load_extension()
    return ext is not None and hasattr(ext, symbol)


def count_launch(n: int = 1) -> None:
    global _launch_count
    _launch_count += n


def launches() -> int:
    return _launch_count


def reset_launches() -> None:
    global _launch_count
    _launch_count = 0
