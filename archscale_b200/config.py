"""Model configuration, the model-name registry and the analytic parameter-count law.

Public surface kept identical to the reference (`lit_gpt/config.py:17-159` for the
dataclass and `from_name`, `:232-265` for `get_parameters_count`, `:267-937` for the
registry): every field name, default and registry key resolves to the same values, so
checkpoints, launch flags and scaling-law scripts written against the reference keep
working.  The registry here is generated from a family table instead of literal dicts.

Fields that do not exist in the reference (expert/tensor-parallel degrees, decoupled
expert sizes, MXFP8) are grouped at the end of the dataclass and default to the
reference behaviour.
"""
from __future__ import annotations

from dataclasses import dataclass, fields
from typing import Any, Dict, Optional

from archscale_b200.utils.misc import find_multiple


@dataclass
class Config:
    org: str = "Microsoft"
    name: str = "transformer_d8"
    block_size: int = 4096
    vocab_size: int = 50254
    padding_multiple: int = 512
    padded_vocab_size: Optional[int] = None
    n_layer: int = 16
    n_head: int = 32
    n_embd: int = 4096
    ar: Optional[int] = None  # aspect ratio: n_embd = ar * n_layer
    mlp_expand: int = 4
    scale_embed: bool = False
    eos_token_id: int = 2
    head_dim: Optional[int] = None
    n_query_groups: Optional[int] = None
    tied_embed: bool = False
    intermediate_size: Optional[int] = None
    # --- MoE ---
    moe: bool = False
    sparsity: int = 1
    top_k: int = 1
    aux_gamma: float = 0.001
    aux_style: str = "switch"  # "entropy" | "switch" | "switch_seq"
    share_expert: bool = False
    zero_mod: bool = False
    sqrt_gate: bool = False
    fuse_sort_and_padding: bool = True
    use_sonicmoe: bool = True
    global_aux: bool = False
    # --- attention ---
    rotary_percentage: float = 1.0
    ada_rope: bool = False
    separate_qkv: bool = True
    fa2: bool = True
    local_window: int = -1
    use_cu_seqlen: bool = False
    qk_norm: bool = False
    attn_norm: bool = False
    nope: bool = False
    sc_attn: bool = False
    use_da: bool = False
    sink_attn: bool = False
    rope_base: int = 10000
    relu2: bool = False
    full_swa_extend: bool = False
    da_const_lamb: bool = False
    use_sigmoid: bool = False
    gated_attn: bool = False
    scaling_factor: float = 1.0
    # --- bias ---
    bias: bool = False
    attn_bias: bool = False
    attn_out_bias: bool = False
    no_mlp_bias: bool = False
    # --- MLP ---
    mlp: bool = True
    oss_swiglu: bool = False
    ffn_norm: bool = False
    mlp_relu2: bool = False
    # --- hybrid ---
    full_per_layer: int = 1000000
    rnn_per_layer: int = -1
    rnn_type: str = "mamba"  # "mamba" | "mamba2" | "gdn" | "retnet" | "gla" | "delta"
    attn_layer_pos: Optional[str] = None
    yoco: bool = False
    gmu_yoco: bool = False
    gmu_per_layer: int = 2
    gmu_attn: bool = False
    gmu_mlp: bool = False
    jamba_norm: bool = False
    yoco_nope: bool = False
    yoco_window: bool = False
    # --- skip connection ---
    post_norm: bool = False
    decouple_postnorm: bool = False
    skip_gain: bool = False
    skip_weight_per_layer: int = -1
    # Residual stream in fp32 instead of the compute dtype.  The reference carries this field (default True, marked deprecated,
    # read nowhere: `lit_gpt/config.py:96`) and adds its residuals in bf16 under bf16 mixed precision (`lit_gpt/model.py:603`);
    # False reproduces that, True keeps the sum of the branches in fp32 at 1.7 % more step time on the dense d16 model.
    residual_in_fp32: bool = False
    no_skip: bool = False
    lc: bool = False
    lc_shared: bool = False
    sc_lc: bool = False
    sum_skip: bool = False
    # --- layer sharing ---
    share_per_layer: int = -1
    share_group: int = 1
    compress: bool = False
    # --- scalers ---
    attn_scale: Optional[float] = None
    w_init_scale: float = 1.0
    # --- scaling rules ---
    head_init_std: Optional[float] = None
    mup_d0: int = 16
    mup: bool = False
    depth_scale: bool = False
    use_muon: bool = False
    use_muonh: bool = False
    super_mup: bool = False
    mup_hd0: int = 128
    shadow_init: bool = False
    original_mup: bool = False
    _norm_class: str = "FusedRMSNorm"
    norm_eps: float = 1e-5
    lc_budget_tau: float = 0.25
    lc_budget_lambda: float = 0.01
    # --- additions of this framework (None / 1 / False = reference behaviour) ---
    n_routed_experts: Optional[int] = None       # routed expert count; default sparsity*top_k (-1 if shared)
    router_top_k: Optional[int] = None           # experts chosen per token; default top_k (-1 if shared)
    moe_intermediate_size: Optional[int] = None  # hidden width of each routed expert; default I/top_k
    shared_intermediate_size: Optional[int] = None  # hidden width of the shared expert; default = routed
    ep_size: int = 1   # expert-parallel degree (experts sharded over this many ranks)
    tp_size: int = 1   # tensor-parallel degree
    mxfp8: bool = False  # E4M3 values + E8M0 scale per 32 elements on every Linear except lm_head
    nvfp4: bool = False  # e2m1 values + E4M3 scale per 16 elements + one fp32 scale per tensor, same layers

    def __post_init__(self) -> None:
        if self.padded_vocab_size is None:
            self.padded_vocab_size = find_multiple(self.vocab_size, self.padding_multiple)
        if self.n_query_groups is not None:
            assert self.n_head % self.n_query_groups == 0
        else:
            self.n_query_groups = self.n_head
        explicit_intermediate = self.intermediate_size is not None
        if not explicit_intermediate:
            self.intermediate_size = self.mlp_expand * self.n_embd
        if self.ar is not None:
            self.n_embd = self.ar * self.n_layer
            # The reference recomputes the MLP width from `ar` unconditionally
            # (lit_gpt/config.py:139-141).  An explicitly passed intermediate_size is an
            # override a benchmark shape needs (e.g. 5632), so it wins here.
            if not explicit_intermediate:
                self.intermediate_size = self.mlp_expand * self.n_embd
        if self.sparsity > 1:
            self.lc_budget_tau = 1 / self.sparsity
        assert self.n_embd % self.n_head == 0 or self.head_dim is not None

    # -- derived quantities -------------------------------------------------------
    @property
    def head_size(self) -> int:
        return self.head_dim if self.head_dim is not None else self.n_embd // self.n_head

    @property
    def total_experts(self) -> int:
        return self.sparsity * self.top_k

    @property
    def routed_experts(self) -> int:
        if self.n_routed_experts is not None:
            return self.n_routed_experts
        return self.total_experts - (1 if self.share_expert else 0)

    @property
    def routed_top_k(self) -> int:
        if self.router_top_k is not None:
            return self.router_top_k
        return self.top_k - (1 if self.share_expert else 0)

    @property
    def expert_hidden(self) -> int:
        if self.moe_intermediate_size is not None:
            return self.moe_intermediate_size
        return self.intermediate_size // self.top_k

    @property
    def shared_hidden(self) -> int:
        if self.shared_intermediate_size is not None:
            return self.shared_intermediate_size
        return self.expert_hidden

    @property
    def norm_class(self):
        from archscale_b200.models import norms

        return norms.norm_class_by_name(self._norm_class)

    @classmethod
    def from_name(cls, name: str, **overrides: Any) -> "Config":
        conf = dict(name_to_config[name])
        conf.update(overrides)
        return cls(**conf)

    def to_dict(self) -> Dict[str, Any]:
        return {f.name: getattr(self, f.name) for f in fields(self)}


# ---------------------------------------------------------------------------------
# Parameter-count law used for the token budget (reference lit_gpt/config.py:232-265)
# ---------------------------------------------------------------------------------
_N_MULT_RULES = (
    # (substring, quadratic coeff, linear coeff); later matches override earlier ones
    ("samba", 15.0, 160.0),
    ("sambay", 14.5, 144.0),
    ("phi4miniflash", 14.5, 144.0),
    ("sambayoco", 13.5, 208.0),
    ("sambayattn", 13.5, 208.0),
    ("mambay", 16.0, 64.0),
    ("gdny", 16.0, 64.0),
    ("sambaymlp", 15.5, 144.0),
    ("swayoco", 12.0, 288.0),
    ("transformer", 12.0, 0.0),
)


def get_parameters_count(model_name: str, depth: int, model_config: Config, train_config: str) -> float:
    """Analytic non-embedding parameter count N(depth) = n_mult * depth^3 (+ corrections)."""
    ar = model_config.ar
    quad, lin = 14.5, 0.0
    for key, q, l in _N_MULT_RULES:
        if key in model_name:
            quad, lin = q, l
    n = (quad * ar * ar + lin * ar) * depth ** 3
    if "v2scale" in train_config:
        emb = depth * ar * model_config.vocab_size
        tied = "_tie" in train_config or model_config.tied_embed
        n += emb if tied else 2 * emb
    if model_config.skip_weight_per_layer > 0:
        n += model_config.n_embd ** 2 * depth // model_config.skip_weight_per_layer
    if "transformer" in model_name:
        hs = model_config.head_size
        n += ar * depth ** 2 * model_config.n_head * hs * 2          # q and o projections
        n += ar * depth ** 2 * model_config.n_query_groups * hs * 2  # k and v projections
    return n


# ---------------------------------------------------------------------------------
# Registry.  Each family is (name template, per-depth field function).
# ---------------------------------------------------------------------------------
_DEPTHS = (8, 12, 16, 20, 24)
_POW2 = (1, 2, 4, 8, 16, 32, 64)
_BASE = dict(org="Microsoft", block_size=4096, vocab_size=32000, padding_multiple=64, mlp_expand=4)
_SAMBAY = dict(rnn_per_layer=2, rnn_type="mamba", yoco=True, gmu_yoco=True, nope=True, head_dim=128, local_window=128)


def _mk(name: str, **kw: Any) -> Dict[str, Any]:
    d = dict(_BASE)
    d["name"] = name
    d.update(kw)
    return d


def _build_registry() -> Dict[str, Dict[str, Any]]:
    reg: Dict[str, Dict[str, Any]] = {}

    def add(entry: Dict[str, Any]) -> None:
        reg[entry["name"]] = entry

    add(_mk("phi4miniflash_d32", block_size=8192, vocab_size=200064, rnn_per_layer=2, rnn_type="mamba", yoco=True,
            gmu_yoco=True, nope=True, attn_bias=True, attn_out_bias=True, n_layer=32, n_head=40, use_da=True,
            head_dim=64, ar=80, tied_embed=True, _norm_class="LayerNorm", n_query_groups=20, local_window=512))

    for d in _DEPTHS:
        q4 = d // 4
        # plain transformer families
        add(_mk(f"transformersa_d{d}", n_layer=d, n_head=d, ar=128, n_query_groups=q4, sink_attn=True))
        add(_mk(f"transformer_d{d}", n_layer=d, n_head=d, ar=128, n_query_groups=q4))
        add(_mk(f"transformer_mha_d{d}", n_layer=d, n_head=d, ar=128, n_query_groups=d))
        add(_mk(f"transformer_gqa4_d{d}", n_layer=d, n_head=d, ar=128, n_query_groups=4))
        add(_mk(f"transformer_gqa4_h2_d{d}", n_layer=d, n_head=2 * d, head_dim=128, ar=128, n_query_groups=4))
        add(_mk(f"transformer_gqa4_h2_skipw_d{d}", skip_weight_per_layer=4, n_layer=d, n_head=2 * d, head_dim=128,
                ar=128, n_query_groups=4))
        add(_mk(f"transformer_gqa4_w8_d{d}", n_layer=d, n_head=d, ar=128, n_query_groups=4, mlp_expand=32))
        add(_mk(f"transformerga_gqa4_d{d}", n_layer=d, n_head=d, ar=124, gated_attn=True, n_query_groups=4))
        add(_mk(f"transformerls_d{d}", full_per_layer=4, n_layer=d, n_head=d, ar=128, n_query_groups=q4,
                local_window=128))
        # hybrids
        add(_mk(f"samba_d{d}", rnn_per_layer=2, rnn_type="mamba", n_layer=d, n_head=d, head_dim=128, ar=122,
                n_query_groups=q4, local_window=2048))
        add(_mk(f"swayoco_d{d}", yoco=True, n_layer=d, n_head=d, head_dim=128, ar=130, n_query_groups=q4,
                local_window=128))
        yw = dict(_SAMBAY, yoco_window=True, n_layer=d, n_head=d, ar=124, n_query_groups=q4)
        wr = dict(yw)
        wr.pop("nope")
        add(_mk(f"sambaywr_d{d}", **wr))
        add(_mk(f"sambaywdr_d{d}", ada_rope=True, **wr))
        add(_mk(f"sambayw_d{d}", **yw))
        add(_mk(f"sambaywsa_d{d}", sink_attn=True, **yw))
        sy = dict(_SAMBAY, n_layer=d, n_head=d, ar=124, n_query_groups=q4)
        add(_mk(f"sambay_d{d}", **sy))
        add(_mk(f"sambayda_d{d}", use_da=True, **sy))
        add(_mk(f"sambayoco_d{d}", **dict(sy, gmu_yoco=False, ar=126)))
        # MoE families
        for k in _POW2:
            for s in _POW2:
                moe = dict(moe=True, top_k=k, sparsity=s)
                add(_mk(f"transformer_gqa4_h2_moe_s{s}_k{k}_d{d}", n_layer=d, n_head=2 * d, head_dim=128, ar=128,
                        n_query_groups=4, **moe))
                add(_mk(f"transformer_gqa4_h2_skipw_moe_s{s}_k{k}_d{d}", skip_weight_per_layer=4, n_layer=d,
                        n_head=2 * d, head_dim=128, ar=128, n_query_groups=4, **moe))
                if k <= 8:
                    add(_mk(f"sambay_gqa4_moe_s{s}_k{k}_d{d}", **dict(_SAMBAY, n_layer=d, n_head=d, ar=124,
                                                                        n_query_groups=4), **moe))
                    add(_mk(f"transformer_gqa4_moe_s{s}_k{k}_d{d}", n_layer=d, n_head=d, ar=128, n_query_groups=4,
                            **moe))

    # fixed-depth ablations (depth 16)
    ab = dict(_SAMBAY, n_layer=16, n_head=16, n_query_groups=4)
    add(_mk("mambay_d16", **dict(ab, rnn_per_layer=1, ar=120)))
    add(_mk("mambay2_d16", **dict(ab, rnn_per_layer=1, rnn_type="mamba2", ar=120)))
    add(_mk("gdny_d16", **dict(ab, rnn_per_layer=1, rnn_type="gdn", ar=120)))
    add(_mk("sgdny_d16", **dict(ab, rnn_type="gdn", ar=126)))
    add(_mk("sambay2_d16", **dict(ab, rnn_type="mamba2", ar=124)))
    add(_mk("sambayattn_d16", **dict(ab, gmu_attn=True, ar=126)))
    add(_mk("sambayattnall_d16", **dict(ab, gmu_attn=True, gmu_per_layer=1, ar=126)))
    add(_mk("sambaymlp_d16", **dict(ab, gmu_mlp=True, ar=120)))
    return reg


name_to_config: Dict[str, Dict[str, Any]] = _build_registry()
configs = list(name_to_config.values())
