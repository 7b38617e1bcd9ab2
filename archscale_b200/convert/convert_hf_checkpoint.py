"""CLI: Hugging Face Llama-style folder (``*.bin`` / ``*.safetensors``) → lit checkpoint ``lit_model.pth``.

    python -m archscale_b200.convert.convert_hf_checkpoint --checkpoint_dir hf_dir --model_name transformer_gqa4_d16
"""
from __future__ import annotations

import argparse
import glob
import os

import torch

from archscale_b200.config import Config
from archscale_b200.convert.hf import hf_to_lit


def _load_hf_dir(path: str) -> dict:
    weights: dict = {}
    files = sorted(glob.glob(os.path.join(path, "*.safetensors")))
    if files:
        from safetensors.torch import load_file
        for f in files:
            weights.update(load_file(f))
        return weights
    for f in sorted(glob.glob(os.path.join(path, "*.bin"))):
        weights.update(torch.load(f, map_location="cpu", weights_only=True))
    if not weights:
        raise FileNotFoundError(f"no *.safetensors or *.bin under {path}")
    return weights


def convert(checkpoint_dir: str, model_name: str, dtype: str = "bfloat16", **overrides) -> str:
    config = Config.from_name(model_name, **overrides)
    lit = {k: v.to(getattr(torch, dtype)).contiguous() for k, v in hf_to_lit(_load_hf_dir(checkpoint_dir), config).items()}
    out = os.path.join(checkpoint_dir, "lit_model.pth")
    torch.save({"model": lit}, out)
    return out


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--checkpoint_dir", required=True)
    ap.add_argument("--model_name", required=True)
    ap.add_argument("--dtype", default="bfloat16")
    a = ap.parse_args()
    print(convert(a.checkpoint_dir, a.model_name, a.dtype))


if __name__ == "__main__":
    main()
