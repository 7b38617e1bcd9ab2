"""Registry parity with the reference and the parameter-count law."""
import os
import re

import pytest

from archscale_b200.config import Config, get_parameters_count, name_to_config

REF = os.path.join(os.environ.get("ARCHSCALE_REFERENCE_DIR", ""), "lit_gpt", "config.py")   # unset → the parity tests skip


def _reference_registry():
    src = open(REF).read()
    start = src.index("configs=[]")
    ns = {}
    exec(src[start:], ns)  # the registry part is plain dict literals / comprehensions
    return ns["name_to_config"]


@pytest.mark.skipif(not os.path.exists(REF), reason="reference tree not mounted")
def test_registry_matches_reference_exactly():
    ref = _reference_registry()
    assert set(ref) == set(name_to_config)
    for name, entry in ref.items():
        assert entry == name_to_config[name], name


def test_registry_size_and_known_entries():
    assert len(name_to_config) == 869
    c = Config.from_name("transformer_gqa4_h2_moe_s8_k8_d8")
    assert (c.n_embd, c.n_head, c.n_query_groups, c.head_size, c.intermediate_size) == (1024, 16, 4, 128, 4096)
    assert c.moe and c.total_experts == 64 and c.expert_hidden == 512
    c = Config.from_name("transformer_gqa4_h2_moe_s8_k8_d8", share_expert=True)
    assert c.routed_experts == 63 and c.routed_top_k == 7
    p = Config.from_name("phi4miniflash_d32")
    assert (p.n_embd, p.padded_vocab_size, p.head_size, p._norm_class) == (2560, 200064, 64, "LayerNorm")


def test_overrides_reach_benchmark_shapes():
    c = Config.from_name("transformer_gqa4_d16", intermediate_size=5632, qk_norm=True)
    assert (c.n_embd, c.n_head, c.n_query_groups, c.head_size, c.intermediate_size) == (2048, 16, 4, 128, 5632)
    m = Config.from_name("transformer_gqa4_h2_moe_s8_k8_d8", n_head=8, n_query_groups=2, n_routed_experts=64,
                         router_top_k=8, moe_intermediate_size=256, shared_intermediate_size=2048, share_expert=True)
    assert (m.routed_experts, m.routed_top_k, m.expert_hidden, m.shared_hidden) == (64, 8, 256, 2048)


def test_parameter_law():
    c8 = Config.from_name("transformer_gqa4_d8")
    n = get_parameters_count("transformer_gqa4_d8", 8, c8, "scaling_mup")
    expect = 12 * 128 ** 2 * 8 ** 3 + 128 * 64 * 8 * 128 * 2 + 128 * 64 * 4 * 128 * 2
    assert n == expect
    s = Config.from_name("sambay_d8")
    assert get_parameters_count("sambay_d8", 8, s, "x") == (14.5 * 124 ** 2 + 144 * 124) * 512
    assert get_parameters_count("sambayoco_d8", 8, Config.from_name("sambayoco_d8"), "x") == (13.5 * 126 ** 2 + 208 * 126) * 512
    v2 = get_parameters_count("transformer_gqa4_d8", 8, c8, "v2scale")
    assert v2 == expect + 2 * 8 * 128 * 32000
