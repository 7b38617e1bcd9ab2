"""CLI: lit checkpoint (``iter-*-ckpt.pth`` or a state-dict file) → Hugging Face folder (``model.bin`` + ``config.json``).

    python -m archscale_b200.convert.convert_lit_checkpoint --checkpoint out/.../iter-001000-ckpt.pth \
        --model_name transformer_gqa4_d16 --output_dir hf_out
"""
from __future__ import annotations

import argparse
import json
import os

import torch

from archscale_b200.config import Config
from archscale_b200.convert.hf import hf_config_from_lit, lit_to_hf


def convert(checkpoint: str, model_name: str, output_dir: str, **overrides) -> str:
    state = torch.load(checkpoint, map_location="cpu", weights_only=False)
    model = state.get("model", state)
    config = Config.from_name(model_name, **overrides)
    hf = {k: v.to(torch.bfloat16).contiguous() for k, v in lit_to_hf(model, config).items()}
    os.makedirs(output_dir, exist_ok=True)
    torch.save(hf, os.path.join(output_dir, "pytorch_model.bin"))
    with open(os.path.join(output_dir, "config.json"), "w") as f:
        json.dump(hf_config_from_lit(config), f, indent=1)
    return output_dir


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--checkpoint", required=True)
    ap.add_argument("--model_name", required=True)
    ap.add_argument("--output_dir", required=True)
    a = ap.parse_args()
    print(convert(a.checkpoint, a.model_name, a.output_dir))


if __name__ == "__main__":
    main()
