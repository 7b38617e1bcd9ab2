"""Checkpoint utilities: averaging of lit checkpoints and MoE parameter accounting.

* ``average_checkpoints`` — arithmetic mean of ``state["model"]`` over several checkpoints; every other entry
  (optimizer state, counters) is taken from the first file (role of `scripts/average_ckpts.py:17-74`).
* ``count_moe_params`` — total vs. active parameters of a built model, by walking its modules instead of the
  closed-form table of `scripts/count_moe_params.py:21-55` (so it stays right for shared experts and hybrids).

    python -m archscale_b200.utils.ckpt_tools average --inputs a.pth b.pth --output avg.pth
    python -m archscale_b200.utils.ckpt_tools average --dir out/run --last 5 --output avg.pth
    python -m archscale_b200.utils.ckpt_tools count --model_name transformer_gqa4_h2_moe_s8_k8_d8
"""
from __future__ import annotations

import argparse
import collections
import glob
import os
import re
from typing import Dict, Iterable, List

import torch


def average_checkpoints(paths: Iterable[str]) -> Dict:
    paths = list(paths)
    if not paths:
        raise ValueError("no checkpoints to average")
    sums: "collections.OrderedDict[str, torch.Tensor]" = collections.OrderedDict()
    out_state = None
    dtypes: Dict[str, torch.dtype] = {}
    for path in paths:
        state = torch.load(path, map_location="cpu", weights_only=False)
        model = state["model"]
        if out_state is None:
            out_state = state
            for k, v in model.items():
                dtypes[k] = v.dtype
                sums[k] = v.detach().clone().to(torch.float64 if v.is_floating_point() else v.dtype)
        else:
            if list(model.keys()) != list(sums.keys()):
                raise KeyError(f"{path}: parameter names differ from {paths[0]}")
            for k, v in model.items():
                sums[k] += v.to(sums[k].dtype)
    n = len(paths)
    avg = collections.OrderedDict()
    for k, v in sums.items():
        avg[k] = (v / n).to(dtypes[k]) if v.is_floating_point() else v // n
    out_state["model"] = avg
    return out_state


def last_checkpoints(directory: str, n: int) -> List[str]:
    """The n most recent ``iter-<step>-ckpt.pth`` files of a run directory, oldest first."""
    hits = []
    for p in glob.glob(os.path.join(directory, "iter-*-ckpt.pth")):
        m = re.search(r"iter-(\d+)-ckpt\.pth$", p)
        if m:
            hits.append((int(m.group(1)), p))
    hits.sort()
    if len(hits) < n:
        raise FileNotFoundError(f"{directory} holds {len(hits)} checkpoints, {n} requested")
    return [p for _, p in hits[-n:]]


def count_moe_params(model: torch.nn.Module) -> Dict[str, int]:
    """total / active-per-token parameter counts; expert stacks count ``top_k / n_experts`` of their size as active."""
    from archscale_b200.models.moe import Experts
    total = active = 0
    expert_param_ids = set()
    for mod in model.modules():
        k = getattr(mod, "top_k", None)
        if k is None:
            continue
        for child in mod.children():              # the expert stacks of one MoE layer share its top_k
            if isinstance(child, Experts):
                for p in child.parameters(recurse=False):
                    expert_param_ids.add(id(p))
                    total += p.numel()
                    active += p.numel() * k // p.shape[0]
    seen = set()
    for p in model.parameters():
        if id(p) in expert_param_ids or id(p) in seen:
            continue
        seen.add(id(p))
        total += p.numel()
        active += p.numel()
    return {"total": total, "active": active}


def main() -> None:
    ap = argparse.ArgumentParser()
    sub = ap.add_subparsers(dest="cmd", required=True)
    a = sub.add_parser("average")
    a.add_argument("--inputs", nargs="*", default=[])
    a.add_argument("--dir", default=None)
    a.add_argument("--last", type=int, default=0)
    a.add_argument("--output", required=True)
    c = sub.add_parser("count")
    c.add_argument("--model_name", required=True)
    args = ap.parse_args()
    if args.cmd == "average":
        paths = list(args.inputs) or last_checkpoints(args.dir, args.last)
        torch.save(average_checkpoints(paths), args.output)
        print(f"averaged {len(paths)} checkpoints into {args.output}")
    else:
        from archscale_b200.config import Config
        from archscale_b200.models.gpt import GPT
        with torch.device("meta"):
            model = GPT(Config.from_name(args.model_name))
        print(count_moe_params(model))


if __name__ == "__main__":
    main()
