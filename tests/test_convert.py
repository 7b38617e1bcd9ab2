"""lit ↔ Hugging Face conversion: name round trip and logits parity with transformers' Llama on CPU."""
import pytest
import torch

from archscale_b200.config import Config
from archscale_b200.convert import hf_config_from_lit, hf_to_lit, lit_to_hf
from archscale_b200.models.gpt import GPT


def _tiny():
    cfg = Config.from_name("transformer_gqa4_d8", vocab_size=320, block_size=64, n_layer=2, n_embd=128, n_head=4,
                           n_query_groups=2, head_dim=32, intermediate_size=256)
    torch.manual_seed(0)
    m = GPT(cfg)
    m.reset_parameters() if hasattr(m, "reset_parameters") else None
    with torch.no_grad():
        for p in m.parameters():
            p.normal_(0, 0.05) if p.dim() > 1 else p.uniform_(0.5, 1.5)
    m.compute_dtype = torch.float32
    return cfg, m.float().eval()


def test_round_trip_names_and_values():
    cfg, m = _tiny()
    lit = m.state_dict()
    hf = lit_to_hf(lit, cfg)
    assert "model.layers.1.mlp.gate_proj.weight" in hf and "model.layers.0.self_attn.o_proj.weight" in hf
    back = hf_to_lit(hf, cfg)
    assert set(back) == set(lit)
    for k in lit:
        assert torch.equal(back[k], lit[k]), k


def test_logits_match_transformers_llama():
    transformers = pytest.importorskip("transformers")
    cfg, m = _tiny()
    hc = hf_config_from_lit(cfg)
    hc.pop("architectures"); hc.pop("model_type"); hc.pop("torch_dtype")
    hf_cfg = transformers.LlamaConfig(**hc, attn_implementation="eager")
    hf_model = transformers.LlamaForCausalLM(hf_cfg).float().eval()
    missing, unexpected = hf_model.load_state_dict(lit_to_hf(m.state_dict(), cfg), strict=False)
    assert not unexpected and all("rotary" in k for k in missing)
    ids = torch.randint(0, cfg.vocab_size, (2, 48))
    with torch.no_grad():
        ours = m(ids)
        ours = ours[0] if isinstance(ours, tuple) else ours
        theirs = hf_model(ids).logits
    assert torch.allclose(ours[..., :cfg.vocab_size], theirs[..., :cfg.vocab_size], atol=2e-4, rtol=2e-4), \
        (ours - theirs).abs().max()
