"""Thin collective layer over ``torch.distributed`` that behaves the same on NCCL and gloo.

gloo (the CPU test backend) has no reduce-scatter; it is emulated with all-reduce + slice so
that the FSDP engine, the optimizers and expert parallelism run unchanged on CPU ranks.
The reference has 16 explicit collective call sites (NCCL only, e.g.
`lit_gpt/optim/muon.py:531-535,554-558,623-635`); this module is the single choke point here.
"""
from __future__ import annotations

import datetime
import os
from typing import List, Optional

import torch
import torch.distributed as dist


def is_dist() -> bool:
    return dist.is_available() and dist.is_initialized()


def world_size(group=None) -> int:
    return dist.get_world_size(group) if is_dist() else 1


def rank(group=None) -> int:
    return dist.get_rank(group) if is_dist() else 0


def init_process_group(backend: Optional[str] = None, timeout_s: float = 600.0) -> None:
    """Initialise from the torchrun environment (RANK / WORLD_SIZE / MASTER_ADDR / MASTER_PORT)."""
    if is_dist() or int(os.environ.get("WORLD_SIZE", "1")) <= 1 and "RANK" not in os.environ:
        return
    if backend is None:
        backend = "nccl" if torch.cuda.is_available() else "gloo"
    if backend == "nccl":
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    kwargs = {}
    if backend == "nccl":
        kwargs["device_id"] = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    dist.init_process_group(backend=backend, timeout=datetime.timedelta(seconds=timeout_s), **kwargs)


def _backend(group=None) -> str:
    return dist.get_backend(group)


def all_gather_into(out: torch.Tensor, inp: torch.Tensor, group=None, async_op: bool = False):
    if world_size(group) == 1:
        out.copy_(inp.view_as(out))
        return None
    return dist.all_gather_into_tensor(out, inp, group=group, async_op=async_op)


def reduce_scatter_sum(out: torch.Tensor, inp: torch.Tensor, group=None):
    """out (S,) = Σ_ranks inp[rank·S:(rank+1)·S]."""
    w = world_size(group)
    if w == 1:
        out.copy_(inp.view_as(out))
        return
    if _backend(group) == "gloo":
        tmp = inp.clone()
        dist.all_reduce(tmp, group=group)
        r = dist.get_rank(group)
        out.copy_(tmp.view(w, -1)[r].view_as(out))
        return
    dist.reduce_scatter_tensor(out, inp, group=group)


def all_reduce_sum(t: torch.Tensor, group=None):
    if world_size(group) > 1:
        dist.all_reduce(t, group=group)
    return t


def all_to_all_single(out: torch.Tensor, inp: torch.Tensor, out_splits: Optional[List[int]] = None,
                      in_splits: Optional[List[int]] = None, group=None):
    if world_size(group) == 1:
        out.copy_(inp)
        return
    dist.all_to_all_single(out, inp, out_splits, in_splits, group=group)


def barrier(group=None):
    if world_size(group) > 1:
        dist.barrier(group=group)


def broadcast_object(obj, src: int = 0, group=None):
    if world_size(group) == 1:
        return obj
    box = [obj]
    dist.broadcast_object_list(box, src=src, group=group)
    return box[0]
