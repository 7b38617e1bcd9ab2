"""Checkpoint IO in the lit layout: ``{"model", "optimizer", "hparams", "iter_num", "step_count"}``.

Reference: `utils.py:255-323` (``_fabric_save_anywhere`` / ``_fabric_load_anywhere`` /
``_latest_ckpt_in_dir_anywhere``; remote copies through azcopy / gsutil / aws CLI) and
`pretrain.py:709,1015-1018,1313-1323` (state keys, file name ``iter-{iter:06d}-ckpt.pth``,
``--resume auto``).  ``state["model"]`` is a consolidated state dict with the model's own key
names, so `torch.load(path)["model"]` loads into an unsharded model exactly as the eval
scripts of the reference expect (`eval.py:113-141`).

Additions: atomic writes (tmp + rename), a validity check so that ``resume=auto`` skips a
truncated file, RNG / data-position round-trip for bitwise-exact resume.
"""
from __future__ import annotations

import os
import re
import shutil
import subprocess
import tempfile
from typing import Any, Dict, Optional

import torch

from archscale_b200.parallel import dist_utils as du

_REMOTE = re.compile(r"^(az|gs|s3)://")
_CKPT_RE = re.compile(r"iter-(\d+)-ckpt\.pth$")


def is_remote(path: str) -> bool:
    return bool(_REMOTE.match(path or ""))


def _remote_copy(src: str, dst: str) -> None:
    scheme = (src if is_remote(src) else dst).split("://", 1)[0]
    cmd = {"az": ["azcopy", "copy", src, dst], "gs": ["gsutil", "cp", src, dst], "s3": ["aws", "s3", "cp", src, dst]}[scheme]
    if shutil.which(cmd[0]) is None:
        raise RuntimeError(f"{cmd[0]} is required for {scheme}:// checkpoints but is not installed")
    subprocess.run(cmd, check=True)


def make_dirs(path: str) -> None:
    if not is_remote(path):
        os.makedirs(path, exist_ok=True)


def ckpt_name(iter_num: int) -> str:
    return f"iter-{iter_num:06d}-ckpt.pth"


def save_anywhere(path: str, state: Dict[str, Any], rank: Optional[int] = None) -> None:
    """Rank 0 writes ``state`` (already consolidated) atomically; all ranks meet at a barrier."""
    rank = du.rank() if rank is None else rank
    if rank == 0:
        if is_remote(path):
            with tempfile.TemporaryDirectory() as td:
                local = os.path.join(td, os.path.basename(path))
                torch.save(state, local)
                _remote_copy(local, path)
        else:
            os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
            tmp = path + ".tmp"
            torch.save(state, tmp)
            os.replace(tmp, path)
    du.barrier()


def load_anywhere(path: str, map_location="cpu") -> Dict[str, Any]:
    if is_remote(path):
        with tempfile.TemporaryDirectory() as td:
            local = os.path.join(td, os.path.basename(path))
            _remote_copy(path, local)
            return torch.load(local, map_location=map_location, weights_only=False)
    return torch.load(path, map_location=map_location, weights_only=False)


def is_valid_checkpoint(path: str) -> bool:
    """A torch zip checkpoint is readable only if its central directory was fully written."""
    try:
        import zipfile
        with zipfile.ZipFile(path) as z:
            return z.testzip() is None
    except Exception:
        return False


def latest_ckpt_in_dir(directory: str, validate: bool = True) -> Optional[str]:
    """Newest (highest iteration) valid ``iter-*-ckpt.pth`` in ``directory`` or None."""
    if is_remote(directory) or not os.path.isdir(directory):
        return None
    found = []
    for f in os.listdir(directory):
        m = _CKPT_RE.search(f)
        if m:
            found.append((int(m.group(1)), os.path.join(directory, f)))
    for _, p in sorted(found, reverse=True):
        if not validate or is_valid_checkpoint(p):
            return p
    return None


def find_resume_path(resume, out_dir: str) -> Optional[str]:
    """``resume`` ∈ {False, True, "auto", path} (reference `pretrain.py:1313-1323`)."""
    if not resume or (isinstance(resume, str) and resume != "auto"):
        return resume or None
    p = latest_ckpt_in_dir(out_dir)
    if resume is True and p is None:
        raise FileNotFoundError(f"--resume=True but no checkpoint found in {out_dir}")
    return p
