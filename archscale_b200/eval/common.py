"""Model loading and generation shared by the evaluation entry points.

* ``config_from_checkpoint_path`` recovers run-time switches from the checkpoint path the trainer wrote
  (``_mup_``, ``_tie``, ``_rbase_``, ``_swa<N>``, ``_ctx<N>`` with the matching RoPE scaling factor) — the
  convention of `eval.py:113-141`.
* ``ModelWrapper.generate`` is token-by-token decoding that re-runs the whole prefix each step (no KV cache),
  greedy or sampled, with EOS and external stopping criteria (`eval.py:36-111`).
"""
from __future__ import annotations

import re
from typing import Callable, Optional, Sequence

import torch
import torch.nn.functional as F

from archscale_b200.config import Config
from archscale_b200.models.gpt import GPT


def config_from_checkpoint_path(checkpoint_path: str, config_name: str) -> Config:
    config = Config.from_name(config_name)
    config.mup = "_mup_" in checkpoint_path
    config.tied_embed = "_tie" in checkpoint_path
    config.rope_base = 640000 if "_rbase_" in checkpoint_path else 10000
    m = re.search(r"_swa(\d+)", checkpoint_path)
    if m:
        config.local_window = int(m.group(1))
    m = re.search(r"_ctx(\d+)", checkpoint_path)
    if m:
        ctx = int(m.group(1))
        config.block_size = ctx
        config.scaling_factor = ctx / (8192 if config.yoco_window else 4096)
    return config


class GenerateOutput:
    def __init__(self, sequences, input_ids, attention_mask):
        self.sequences, self.input_ids, self.attention_mask = sequences, input_ids, attention_mask


class ModelWrapper(torch.nn.Module):
    def __init__(self, model: GPT) -> None:
        super().__init__()
        self.model = model
        self.config = model.config

    @property
    def device(self) -> torch.device:
        return next(self.model.parameters()).device

    def forward(self, input_ids: torch.Tensor, attention_mask: Optional[torch.Tensor] = None, **kwargs):
        return self.model(input_ids, attn_mask=attention_mask, **kwargs)

    @torch.no_grad()
    def generate(self, input_ids: torch.Tensor, attention_mask: Optional[torch.Tensor] = None, max_length: Optional[int] = None,
                 return_dict_in_generate: bool = True, pad_token_id: Optional[int] = None, eos_token_id: Optional[int] = None,
                 do_sample: bool = False, temperature: Optional[float] = None,
                 stopping_criteria: Optional[Sequence[Callable]] = None, max_gen_toks: int = 128, **_unused):
        sequences = input_ids.clone()
        max_new = max_length - input_ids.shape[1] if max_length else max_gen_toks
        if attention_mask is None:
            attention_mask = (input_ids != pad_token_id).long() if pad_token_id is not None else torch.ones_like(input_ids)
        use_mask = bool((attention_mask == 0).any())
        active = torch.ones(input_ids.shape[0], dtype=torch.bool, device=input_ids.device)
        for _ in range(max(max_new, 0)):
            logits = self.model(sequences, attn_mask=attention_mask if use_mask else None).logits[:, -1, :].float()
            if do_sample:
                if temperature is not None and temperature > 0:
                    logits = logits / float(temperature)
                nxt = torch.multinomial(F.softmax(logits, dim=-1), num_samples=1)
            else:
                nxt = logits.argmax(dim=-1, keepdim=True)
            sequences = torch.cat([sequences, nxt], dim=-1)
            attention_mask = torch.cat([attention_mask, torch.ones_like(nxt)], dim=-1)
            if stopping_criteria is not None and any(bool(torch.as_tensor(c(sequences, None)).all()) for c in stopping_criteria):
                break
            if eos_token_id is not None:
                active = active & (nxt.squeeze(-1) != eos_token_id)
                if not active.any():
                    break
        if return_dict_in_generate:
            return GenerateOutput(sequences, input_ids, attention_mask)
        return sequences


def load_model(checkpoint_path: str, config_name: str, device="cuda", dtype=torch.bfloat16) -> ModelWrapper:
    config = config_from_checkpoint_path(checkpoint_path, config_name)
    model = GPT(config)
    state = torch.load(checkpoint_path, map_location="cpu", weights_only=False)
    model.load_state_dict(state.get("model", state))
    model.to(device=device, dtype=dtype)
    model.compute_dtype = dtype
    model.eval()
    return ModelWrapper(model)
