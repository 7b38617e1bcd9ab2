"""Weight-name and layout maps between the lit checkpoint layout and Hugging Face Llama/Qwen3-style names.

Role of `scripts/convert_hf_checkpoint.py:118-177` and `scripts/convert_lit_checkpoint.py:176-218,263-279`
in the reference, rewritten for the parameter names the current model uses (separate ``q_proj/k_proj/v_proj``,
fused gate+up ``mlp.w1`` with the gate rows first, down projection ``mlp.w3``); the reference scripts still
target the older fused ``attn.attn.weight`` / ``mlp.swiglu.w1/w2/w3`` names and do not load current checkpoints.

Only dense transformer blocks have a Hugging Face counterpart; hybrid (Mamba / GMU / YOCO) and MoE checkpoints
stay in the lit layout.
"""
from __future__ import annotations

import re
from typing import Dict

import torch

from archscale_b200.config import Config

_LAYER = re.compile(r"^(model\.layers|transformer\.h)\.(\d+)\.(.+)$")

_HF_TO_LIT_LAYER = {
    "input_layernorm.weight": "norm_1.weight",
    "input_layernorm.bias": "norm_1.bias",
    "post_attention_layernorm.weight": "norm_2.weight",
    "post_attention_layernorm.bias": "norm_2.bias",
    "self_attn.q_proj.weight": "attn.q_proj.weight",
    "self_attn.k_proj.weight": "attn.k_proj.weight",
    "self_attn.v_proj.weight": "attn.v_proj.weight",
    "self_attn.q_proj.bias": "attn.q_proj.bias",
    "self_attn.k_proj.bias": "attn.k_proj.bias",
    "self_attn.v_proj.bias": "attn.v_proj.bias",
    "self_attn.o_proj.weight": "attn.proj.weight",
    "self_attn.o_proj.bias": "attn.proj.bias",
    "self_attn.q_norm.weight": "attn.q_norm.weight",
    "self_attn.k_norm.weight": "attn.k_norm.weight",
    "mlp.down_proj.weight": "mlp.w3.weight",
}
_LIT_TO_HF_LAYER = {v: k for k, v in _HF_TO_LIT_LAYER.items()}
_HF_TO_LIT_TOP = {"model.embed_tokens.weight": "transformer.wte.weight", "model.norm.weight": "transformer.ln_f.weight",
                  "model.norm.bias": "transformer.ln_f.bias", "lm_head.weight": "lm_head.weight"}
_LIT_TO_HF_TOP = {v: k for k, v in _HF_TO_LIT_TOP.items()}


def hf_to_lit(hf: Dict[str, torch.Tensor], config: Config) -> Dict[str, torch.Tensor]:
    """Hugging Face Llama-style state dict → lit state dict of :class:`archscale_b200.models.gpt.GPT`."""
    out: Dict[str, torch.Tensor] = {}
    gate: Dict[int, torch.Tensor] = {}
    up: Dict[int, torch.Tensor] = {}
    for name, t in hf.items():
        if name.endswith("rotary_emb.inv_freq"):
            continue
        m = _LAYER.match(name)
        if m is None:
            if name not in _HF_TO_LIT_TOP:
                raise KeyError(f"no lit counterpart for {name}")
            out[_HF_TO_LIT_TOP[name]] = t
            continue
        i, rest = int(m.group(2)), m.group(3)
        if rest == "mlp.gate_proj.weight":
            gate[i] = t
        elif rest == "mlp.up_proj.weight":
            up[i] = t
        elif rest in _HF_TO_LIT_LAYER:
            out[f"transformer.h.{i}.{_HF_TO_LIT_LAYER[rest]}"] = t
        else:
            raise KeyError(f"no lit counterpart for {name}")
    for i in sorted(gate):
        out[f"transformer.h.{i}.mlp.w1.weight"] = torch.cat([gate[i], up[i]], dim=0)   # gate rows first
    if config.tied_embed:
        out.pop("lm_head.weight", None)
    elif "lm_head.weight" not in out:
        out["lm_head.weight"] = out["transformer.wte.weight"]
    return out


def lit_to_hf(lit: Dict[str, torch.Tensor], config: Config) -> Dict[str, torch.Tensor]:
    """lit state dict (``state["model"]`` of a checkpoint) → Hugging Face Llama-style names."""
    out: Dict[str, torch.Tensor] = {}
    for name, t in lit.items():
        m = _LAYER.match(name)
        if m is None:
            if name not in _LIT_TO_HF_TOP:
                raise KeyError(f"no Hugging Face counterpart for {name}")
            out[_LIT_TO_HF_TOP[name]] = t
            continue
        i, rest = int(m.group(2)), m.group(3)
        if rest == "mlp.w1.weight":
            g, u = t.chunk(2, dim=0)
            out[f"model.layers.{i}.mlp.gate_proj.weight"] = g
            out[f"model.layers.{i}.mlp.up_proj.weight"] = u
        elif rest in _LIT_TO_HF_LAYER:
            out[f"model.layers.{i}.{_LIT_TO_HF_LAYER[rest]}"] = t
        else:
            raise KeyError(f"{name}: only dense transformer blocks convert to the Hugging Face layout")
    if "lm_head.weight" not in out:
        out["lm_head.weight"] = out["model.embed_tokens.weight"]
    return out


def hf_config_from_lit(config: Config) -> dict:
    """``config.json`` fields of a LlamaForCausalLM equivalent (`scripts/convert_lit_checkpoint.py:263-279`)."""
    return {
        "architectures": ["LlamaForCausalLM"], "model_type": "llama",
        "vocab_size": config.padded_vocab_size, "hidden_size": config.n_embd, "num_hidden_layers": config.n_layer,
        "num_attention_heads": config.n_head, "num_key_value_heads": config.n_query_groups,
        "head_dim": config.head_size, "intermediate_size": config.intermediate_size,
        "max_position_embeddings": config.block_size, "rms_norm_eps": config.norm_eps,
        "rope_theta": float(getattr(config, "rope_base", 10000)), "hidden_act": "silu",
        "tie_word_embeddings": bool(config.tied_embed), "attention_bias": bool(config.attn_bias), "mlp_bias": False,
        "torch_dtype": "bfloat16",
    }
