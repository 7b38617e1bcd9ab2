"""GPT: embeddings → N × Block (token mixer + MLP/MoE) → final norm → head / FLCE hand-off.

Reference: `lit_gpt/model.py:101-351` (``GPT``: constructor, ``reset_parameters`` with the
μP++ head rule / GPT-2 out-projection scaling / ``w_init_scale``, ``forward`` returning
``CausalLMOutput(logits, weight)``), `:354-605` (``Block``: YOCO / SambaY layer map, pre/post
norm, residual stream, depth scaling) and `:620-677` (``LLaMAMLP`` with fused
``w1 = [gate; up]`` and ``w3`` down projection).  Module and parameter names are unchanged
because they are the checkpoint format.

What differs: no ``torch.compile``; every hot op is an explicit call into
:mod:`archscale_b200.ops`; per-layer activation statistics are only computed when
``collect_stats`` is on (the trainer enables it on logging steps) instead of on every forward;
packed-document metadata (``cu_seqlens`` / ``seq_idx``) is computed once per forward, on the
device, instead of once per layer.
"""
from __future__ import annotations

import copy
import math
from typing import Any, List, NamedTuple, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from archscale_b200 import ops
from archscale_b200.config import Config
from archscale_b200.models.attention import CausalSelfAttention
from archscale_b200.models.gated_deltanet import GatedDeltaNet
from archscale_b200.models.gmu import GMUWrapper
from archscale_b200.models.layer_configurator import LayerConfigurator
from archscale_b200.models.layers import Linear
from archscale_b200.models.mamba import Mamba
from archscale_b200.models.mamba2 import Mamba2
from archscale_b200.models.moe import Experts, get_moe
from archscale_b200.models.norms import RMSNormFunc
from archscale_b200.utils.init import torch_default_init


class CausalLMOutput(NamedTuple):
    logits: torch.Tensor
    weight: Optional[torch.Tensor] = None


def mamba2_expand(n_embd: int) -> float:
    return 8 * math.ceil(n_embd * 2 / 64 / 8) * 64 / n_embd


def get_rnn(config: Config, layer_idx: int, gmu_save: bool = False, **factory_kwargs):
    fk = {k: v for k, v in factory_kwargs.items() if k in ("device", "dtype", "jamba_norm")}
    if config.rnn_type == "mamba":
        return Mamba(config.n_embd, layer_idx=layer_idx, gmu_save=gmu_save, config=config, **fk)
    if config.rnn_type == "mamba2":
        return Mamba2(config.n_embd, expand=mamba2_expand(config.n_embd), layer_idx=layer_idx, gmu_save=gmu_save,
                      config=config, **fk)
    if config.rnn_type == "gdn":
        return GatedDeltaNet(hidden_size=config.n_embd, num_heads=math.ceil(int(config.n_embd * 0.75) / 256),
                             head_dim=256, mode="chunk", gmu_save=gmu_save, use_short_conv=True,
                             allow_neg_eigval=True)
    raise ValueError(f"rnn_type {config.rnn_type!r} is not available (supported: mamba, mamba2, gdn); the "
                     "retnet/gla/delta mixers of the reference raise NameError on construction")


def compute_rmsnorm(x: torch.Tensor) -> torch.Tensor:
    return torch.sqrt(torch.mean(x.float() ** 2) + 1e-30)


def compute_outlier_percentage(x: torch.Tensor, sigma: float = 5.0) -> torch.Tensor:
    x = x.float()
    mean, std = x.mean(dim=-1, keepdim=True), x.std(dim=-1, keepdim=True)
    return ((x - mean).abs() > sigma * std).float().mean() * 100.0


def _norm_to(norm: nn.Module, x: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """Apply ``norm`` and deliver ``dtype``; RMSNorm modules convert inside their kernel."""
    from archscale_b200.models.norms import FusedRMSNorm
    if isinstance(norm, FusedRMSNorm):
        return norm(x, out_dtype=dtype)
    return norm(x).to(dtype)


class LLaMAMLP(nn.Module):
    def __init__(self, config: Config) -> None:
        super().__init__()
        self.config = config
        self.relu2 = config.mlp_relu2
        self.oss_swiglu = config.oss_swiglu
        I = config.intermediate_size
        in_size, out_size = (int(I * 1.5), int(I * 1.5)) if self.relu2 else (2 * I, I)
        self.w1 = Linear(config.n_embd, in_size, bias=config.bias)
        self.w3 = Linear(out_size, config.n_embd, bias=config.bias)
        if config.ffn_norm:
            self.norm = config.norm_class(out_size, eps=config.norm_eps)

    def reset_parameters(self) -> None:
        for lin in (self.w1, self.w3):
            torch_default_init(lin.weight)
            if lin.bias is not None:
                nn.init.zeros_(lin.bias)
        if hasattr(self, "norm") and hasattr(self.norm, "reset_parameters"):
            self.norm.reset_parameters()

    def forward(self, x: torch.Tensor, layer_idx: int, gmu_mems=None):
        if (not self.relu2 and not self.oss_swiglu and type(self.w1) is Linear and self.w1.bias is None
                and not self.w1.mxfp8 and not self.w1.nvfp4
                and not (self.config.gmu_mlp and layer_idx == self.config.n_layer // 2 + 1)):
            h = ops.linear_swiglu(x, self.w1.weight)    # SwiGLU in the GEMM epilogue when the kernel takes this case
            if h is not None:
                if self.config.ffn_norm:
                    h = self.norm(h)
                return self.w3(h), gmu_mems
        h = self.w1(x)
        if self.relu2:
            h = F.relu(h).square()
        else:
            if self.config.gmu_mlp and layer_idx == self.config.n_layer // 2 + 1:
                gmu_mems = h[..., h.shape[-1] // 2:]
            if self.oss_swiglu:
                g, u = h.chunk(2, dim=-1)
                h = ops.oss_swiglu_ref(g, u)
            else:
                h = ops.swiglu_packed(h)
        if self.config.ffn_norm:
            h = self.norm(h)
        return self.w3(h), gmu_mems


class Block(nn.Module):
    def __init__(self, config: Config, layer_idx: int) -> None:
        super().__init__()
        self.layer_idx = layer_idx
        self.decouple_scaler = config.decouple_postnorm
        mk_norm = (lambda: RMSNormFunc(config.n_embd, eps=config.norm_eps, decouple_gain=True,
                                       skip_gain=config.skip_gain)) if self.decouple_scaler else \
                  (lambda: config.norm_class(config.n_embd, eps=config.norm_eps))
        self.norm_1 = mk_norm()
        self.use_skip_proj = config.skip_weight_per_layer > 0 and \
            layer_idx % config.skip_weight_per_layer == config.skip_weight_per_layer - 1
        if self.use_skip_proj:
            self.skip_proj = Linear(config.n_embd, config.n_embd, bias=config.bias)
        self.use_rnn = self.use_gmu = self.yoco_kv = self.gmu_save = self.yoco_cross = False
        self.rnn_type = config.rnn_type
        self.last_layer = layer_idx == config.n_layer - 1
        L = config.n_layer
        if config.yoco:
            config = copy.deepcopy(config)
            assert L % 4 == 0, "n_layer should be divisible by 4 for samba + yoco"
            if layer_idx < L // 2:
                self.use_rnn = config.rnn_per_layer > 0 and layer_idx % config.rnn_per_layer == 0
                self.use_full = False
            else:
                self.gmu_save = bool(config.gmu_yoco and not config.gmu_attn)
                self.yoco_kv = layer_idx >= L // 2 + 1
                self.yoco_cross = layer_idx >= L // 2 + 2
                self.use_full = layer_idx >= L // 2 + 1
                if layer_idx == L // 2:
                    self.use_rnn = config.rnn_per_layer > 0
                if config.gmu_yoco and layer_idx >= L // 2 + 2:
                    self.use_gmu = layer_idx % config.gmu_per_layer == 0
            if self.use_full:
                config.local_window = config.block_size // 2 if config.yoco_window else -1
        elif config.attn_layer_pos is not None:
            positions = [int(p) for p in str(config.attn_layer_pos).strip("[]() ").split(",") if p.strip()]
            self.use_rnn = layer_idx not in positions
        else:
            self.use_rnn = config.rnn_per_layer > 0 and layer_idx % config.rnn_per_layer == 0

        if self.use_gmu:
            if config.gmu_attn:
                gmu_inner = config.head_size * config.n_head
            elif config.gmu_mlp:
                gmu_inner = config.intermediate_size
            elif config.rnn_per_layer > 0 and config.rnn_type == "mamba2":
                gmu_inner = int(config.n_embd * mamba2_expand(config.n_embd))
            elif config.rnn_per_layer > 0 and config.rnn_type == "gdn":
                gmu_inner = math.ceil(int(config.n_embd * 0.75) / 256) * 256 * 2
            else:
                gmu_inner = config.n_embd * 2
            use_norm = config.rnn_per_layer > 0 and config.rnn_type in ("mamba2", "gdn")
            self.attn = GMUWrapper(config.n_embd, gmu_inner, bias=config.bias, use_norm=use_norm)
        elif self.use_rnn:
            self.attn = get_rnn(config, layer_idx, gmu_save=self.gmu_save, jamba_norm=config.jamba_norm,
                                dtype=torch.float32)
        else:
            if config.relu2:
                raise NotImplementedError("relu2 attention has no registry entry and is not provided")
            self.attn = CausalSelfAttention(config, n_embd=config.n_embd, layer_idx=layer_idx,
                                            yoco_cross=self.yoco_cross)
        if config.mlp:
            self.norm_2 = mk_norm()
            self.mlp = get_moe(config, is_attn=False, is_mlp=True) if config.moe else LLaMAMLP(config)
        self.config = config
        if config.lc and not config.lc_shared:
            self.layer_configurator = LayerConfigurator(config)
            if config.mlp:
                self.lc_mlp = LayerConfigurator(config)
        self.collect_stats = False
        self.attn_output_rmsnorm = self.mlp_output_rmsnorm = None
        self.attn_outlier_pct = self.mlp_outlier_pct = None
        self.attn_z_mean = self.router_z_mean = None

    def reset_parameters(self) -> None:
        for n in (self.norm_1, getattr(self, "norm_2", None)):
            if n is not None and hasattr(n, "reset_parameters"):
                n.reset_parameters()
        self.attn.reset_parameters()
        if hasattr(self, "skip_proj"):
            torch_default_init(self.skip_proj.weight)
            if self.skip_proj.bias is not None:
                nn.init.zeros_(self.skip_proj.bias)
        if self.config.mlp:
            self.mlp.reset_parameters()
        for n in ("layer_configurator", "lc_mlp"):
            if hasattr(self, n):
                getattr(self, n).reset_parameters()

    # -- helpers -------------------------------------------------------------------
    def _stream_dtype(self, compute_dtype: torch.dtype) -> torch.dtype:
        """Type of the residual stream: fp32 (``residual_in_fp32``), else the compute dtype — what the reference's bf16 mixed
        precision amounts to, where ``x = ox + h`` (`lit_gpt/model.py:603`) adds two bf16 tensors."""
        return torch.float32 if self.config.residual_in_fp32 else compute_dtype

    def _norm_in(self, norm, x, compute_dtype):
        """Returns (residual stream ox, mixer input n)."""
        if self.config.post_norm:
            ox = x.to(norm.weight.dtype) if hasattr(norm, "weight") else x
            ox = norm(ox).to(compute_dtype)
            n = ox * norm.weight if self.decouple_scaler else ox
            if self.config.skip_gain:
                ox = ox * norm.weight1
            return ox, n
        ox = x.to(self._stream_dtype(compute_dtype))
        return ox, norm(x).to(compute_dtype)

    def post_process_residual(self, h, ox, lc, input_embed, residual_dropout: float = 0.0):
        if lc is not None:
            h = lc.extract(h) * torch.sqrt((2 * lc.gate - 1) * lc.act_mask + 1e-5)
        elif self.config.depth_scale:
            h = h / math.sqrt(2 * self.config.n_layer)
        if self.training and residual_dropout > 0:
            h = F.dropout(h, p=residual_dropout, training=True)
        if self.config.no_skip:
            x = h
        elif self.config.sum_skip:
            x = h
            input_embed = input_embed.to(torch.float32) + h.to(torch.float32)
        else:
            x = ox + h
        return x, h, input_embed

    def _deferred_ok(self, x, lc, residual_dropout) -> bool:
        """The fused pre-norm path (residual add deferred into the next norm kernel) applies to the
        standard block: pre-norm RMSNorm with weight, plain skip connection, MLP present, no token skipping."""
        from archscale_b200.models.norms import FusedRMSNorm
        cfg = self.config
        return (x.is_cuda and not cfg.post_norm and not cfg.no_skip and not cfg.sum_skip and cfg.mlp and lc is None
                and not hasattr(self, "layer_configurator") and type(self.norm_1) in (FusedRMSNorm,)
                and type(self.norm_2) in (FusedRMSNorm,) and not (self.training and residual_dropout > 0))

    def forward_deferred(self, x, h_pending, input_embed, rope, max_seq_length, seq_meta, kv_cache, gmu_mems,
                         compute_dtype):
        """Same math as :meth:`forward`; takes the residual stream ``x`` plus the not-yet-added branch
        output ``h_pending`` of the previous block and returns its own MLP output un-added."""
        cfg = self.config
        scale = 1.0 / math.sqrt(2 * cfg.n_layer) if cfg.depth_scale else 1.0
        cu_seqlens = seq_meta.get("cu_seqlens") if seq_meta else None
        seq_idx = seq_meta.get("seq_idx") if seq_meta else None
        pad_mask = seq_meta.get("pad_mask") if seq_meta else None
        stream = self._stream_dtype(compute_dtype)
        x, n_1 = ops.add_rms_norm(x, h_pending, self.norm_1.weight, self.norm_1.eps, scale, compute_dtype, stream)
        new_kv_cache = kv_cache
        if self.use_rnn:
            if self.rnn_type in ("mamba", "mamba2"):
                h, gmu_mems = self.attn(n_1, seq_idx=seq_idx, mask=cu_seqlens if cfg.use_cu_seqlen else pad_mask,
                                        gmu_mems=gmu_mems)
            else:
                h, gmu_mems = self.attn(n_1, attention_mask=None if cfg.use_cu_seqlen else pad_mask,
                                        cu_seqlens=cu_seqlens, gmu_mems=gmu_mems)
        elif self.use_gmu:
            h, gmu_mems = self.attn(n_1, gmu_mems)
        else:
            h, new_kv_cache, gmu_mems = self.attn(n_1, rope, max_seq_length, cu_seqlens, None, kv_cache, gmu_mems)
        if self.collect_stats:
            with torch.no_grad():
                self.attn_output_rmsnorm = compute_rmsnorm(h) * scale
                self.attn_outlier_pct = compute_outlier_percentage(h)
                self.attn_z_mean = getattr(self.attn, "z_mean", None)
        x, n_2 = ops.add_rms_norm(x, h.to(compute_dtype), self.norm_2.weight, self.norm_2.eps, scale, compute_dtype, stream)
        if cfg.moe:
            h = self.mlp(n_2)
        else:
            h, gmu_mems = self.mlp(n_2, self.layer_idx, gmu_mems)
        if self.collect_stats:
            with torch.no_grad():
                self.mlp_output_rmsnorm = compute_rmsnorm(h) * scale
                self.mlp_outlier_pct = compute_outlier_percentage(h)
                self.router_z_mean = getattr(self.mlp, "router_z_mean", None)
        return x, new_kv_cache, gmu_mems, input_embed, h.to(compute_dtype)

    def forward(self, x, input_embed, rope, max_seq_length: int, seq_meta=None, input_pos=None, kv_cache=None,
                lc=None, gmu_mems=None, residual_dropout: float = 0.0, lc_gate_hist=None,
                compute_dtype: torch.dtype = torch.bfloat16, h_pending=None, deferred: bool = False):
        cfg = self.config
        if deferred:
            return self.forward_deferred(x, h_pending, input_embed, rope, max_seq_length, seq_meta, kv_cache, gmu_mems,
                                         compute_dtype)
        cu_seqlens = seq_meta.get("cu_seqlens") if seq_meta else None
        seq_idx = seq_meta.get("seq_idx") if seq_meta else None
        pad_mask = seq_meta.get("pad_mask") if seq_meta else None
        if hasattr(self, "layer_configurator"):
            lc = self.layer_configurator
        ox_src = x
        if lc is not None:
            x = lc(x)
            lc_gate_hist.append(lc.gate if hasattr(self, "layer_configurator") else lc.gate.clone())
        if cfg.post_norm:
            ox, n_1 = self._norm_in(self.norm_1, ox_src, compute_dtype)
            if self.use_skip_proj:
                ox = self.skip_proj(ox)
        else:
            ox = ox_src.to(self._stream_dtype(compute_dtype))
            n_1 = _norm_to(self.norm_1, x, compute_dtype)
        new_kv_cache = kv_cache
        if self.use_rnn:
            if self.rnn_type in ("mamba", "mamba2"):
                mask = cu_seqlens if cfg.use_cu_seqlen else pad_mask
                h, gmu_mems = self.attn(n_1, seq_idx=seq_idx, mask=mask, gmu_mems=gmu_mems)
            else:
                h, gmu_mems = self.attn(n_1, attention_mask=None if cfg.use_cu_seqlen else pad_mask,
                                        cu_seqlens=cu_seqlens, gmu_mems=gmu_mems)
        elif self.use_gmu:
            h, gmu_mems = self.attn(n_1, gmu_mems)
        else:
            h, new_kv_cache, gmu_mems = self.attn(n_1, rope, max_seq_length, cu_seqlens, input_pos, kv_cache, gmu_mems)
        x, h, input_embed = self.post_process_residual(h, ox, lc, input_embed, residual_dropout)
        if self.collect_stats:
            with torch.no_grad():
                self.attn_output_rmsnorm = compute_rmsnorm(h)
                self.attn_outlier_pct = compute_outlier_percentage(h)
                self.attn_z_mean = getattr(self.attn, "z_mean", None)
        if cfg.mlp:
            if hasattr(self, "lc_mlp"):
                lc = self.lc_mlp
            ox_src = x
            if lc is not None:
                x = lc(x)
                lc_gate_hist.append(lc.gate if hasattr(self, "lc_mlp") else lc.gate.clone())
            if cfg.post_norm:
                ox, n_2 = self._norm_in(self.norm_2, ox_src, compute_dtype)
            else:
                ox = ox_src.to(self._stream_dtype(compute_dtype))
                n_2 = _norm_to(self.norm_2, x, compute_dtype)
            if cfg.moe:
                h = self.mlp(n_2)
            else:
                h, gmu_mems = self.mlp(n_2, self.layer_idx, gmu_mems)
            x, h, input_embed = self.post_process_residual(h, ox, lc, input_embed, residual_dropout)
            if self.collect_stats:
                with torch.no_grad():
                    self.mlp_output_rmsnorm = compute_rmsnorm(h)
                    self.mlp_outlier_pct = compute_outlier_percentage(h)
                    self.router_z_mean = getattr(self.mlp, "router_z_mean", None)
        return x, new_kv_cache, gmu_mems, input_embed


class GPT(nn.Module):
    def __init__(self, config: Config) -> None:
        super().__init__()
        assert config.padded_vocab_size is not None
        self.config = config
        self.mup, self.shadow_init, self.super_mup = config.mup, config.shadow_init, config.super_mup
        self.logit_scale = config.mup_d0 / config.n_layer if (config.mup and not config.use_muonh) else 1.0
        self.lm_head = Linear(config.n_embd, config.padded_vocab_size, bias=False)
        block_cfg = config
        if config.lc and config.sparsity > 1:
            block_cfg = copy.deepcopy(config)
            block_cfg.n_layer = config.n_layer * config.sparsity
        num_layer = block_cfg.share_per_layer * block_cfg.share_group if block_cfg.share_per_layer > 0 else block_cfg.n_layer
        if config.moe:
            self.n_attn = [0] * num_layer
            self.n_mlp = [config.sparsity * config.top_k] * num_layer
        self.transformer = nn.ModuleDict(dict(
            wte=nn.Embedding(config.padded_vocab_size, config.n_embd),
            h=nn.ModuleList(Block(block_cfg, i) for i in range(num_layer)),
            ln_f=config.norm_class(config.n_embd, eps=config.norm_eps),
        ))
        self.block_cfg = block_cfg
        self.layer_configurator = LayerConfigurator(block_cfg) if (config.lc and config.lc_shared) else None
        self.lc_gate_hist: List[torch.Tensor] = []
        self.rope_cache = None
        self.max_len = config.block_size
        self.scale_embed, self.tied_embed = config.scale_embed, config.tied_embed
        self.compute_dtype = torch.bfloat16
        self.collect_stats = False
        self.aux_loss: Any = 0.0
        self.tokens_per_expert: list = []
        self.token_indices: list = []
        if self.tied_embed:
            self.tie_weights()

    def tie_weights(self) -> None:
        self.lm_head.weight = self.transformer.wte.weight

    @classmethod
    def from_name(cls, name: str, **kwargs: Any) -> "GPT":
        return cls(Config.from_name(name, **kwargs))

    # -- init ------------------------------------------------------------------------
    @torch.no_grad()
    def reset_parameters(self) -> None:
        cfg = self.config
        std = 0.02 if self.tied_embed else 1e-4
        if self.scale_embed:
            std = std / math.sqrt(cfg.n_embd)
        nn.init.normal_(self.transformer.wte.weight, std=std)
        if not self.tied_embed:
            torch_default_init(self.lm_head.weight)
        if hasattr(self.transformer.ln_f, "reset_parameters"):
            self.transformer.ln_f.reset_parameters()
        for block in self.transformer.h:
            block.reset_parameters()
        if self.layer_configurator is not None:
            self.layer_configurator.reset_parameters()
        n_layer = cfg.n_layer
        if self.mup and not self.tied_embed:
            if cfg.head_init_std is not None:
                nn.init.normal_(self.lm_head.weight, std=cfg.head_init_std)
            else:
                nn.init.zeros_(self.lm_head.weight)
        else:
            per_layer = 2 if cfg.mlp else 1
            for name, p in self.named_parameters():
                if p.requires_grad and name.endswith(("out_proj.weight", "o_proj.weight", "proj.weight", "w3.weight")):
                    p /= math.sqrt(per_layer * n_layer)
        for name, p in self.named_parameters():
            if p.requires_grad and "weight" in name:
                parent = self.get_submodule(name.rsplit(".", 1)[0])
                if isinstance(parent, (nn.Linear, Experts)) or parent.__class__.__name__ == "_PerExpertLinear":
                    if not self.mup:
                        nn.init.normal_(p, std=0.02)
                    p.data *= cfg.w_init_scale
        if self.tied_embed:
            self.tie_weights()

    def set_collect_stats(self, flag: bool) -> None:
        self.collect_stats = flag
        for b in self.transformer.h:
            b.collect_stats = flag
            if hasattr(b.attn, "collect_stats"):
                b.attn.collect_stats = flag
            if hasattr(b, "mlp") and hasattr(b.mlp, "collect_stats"):
                b.mlp.collect_stats = flag

    # -- sequence metadata -------------------------------------------------------------
    def _seq_meta(self, idx: torch.Tensor, attn_mask: Optional[torch.Tensor]):
        cfg = self.config
        if cfg.use_cu_seqlen:
            assert idx.size(0) == 1, "packed variable-length training uses batch size 1"
            is_eos = idx.flatten() == cfg.eos_token_id
            T = idx.shape[1]
            ends = is_eos.nonzero().flatten() + 1
            ends = ends[ends < T]
            cu = torch.cat([ends.new_zeros(1), ends, ends.new_full((1,), T)]).to(torch.int32)
            # document id of each token: number of EOS strictly before it
            seq_idx = (torch.cumsum(is_eos.to(torch.int32), 0) - is_eos.to(torch.int32)).unsqueeze(0).to(torch.int32)
            return {"cu_seqlens": cu, "seq_idx": seq_idx}
        if attn_mask is not None:
            return {"pad_mask": attn_mask}
        return None

    def build_rope_cache(self, idx: torch.Tensor, seq_len: int):
        cfg = self.config
        return ops.build_rope_cache(seq_len, int(cfg.rotary_percentage * cfg.head_size), self.compute_dtype, idx.device,
                                    base=cfg.rope_base, scaling_factor=cfg.scaling_factor)

    # -- forward -------------------------------------------------------------------------
    def forward(self, idx: torch.Tensor, max_seq_length: Optional[int] = None,
                attn_mask: Optional[torch.Tensor] = None, residual_dropout: float = 0.0,
                use_flce_loss: bool = False) -> CausalLMOutput:
        cfg = self.config
        B, T = idx.shape
        seq_meta = self._seq_meta(idx, attn_mask)
        if max_seq_length is None:
            max_seq_length = cfg.block_size
        rope = None
        if not (cfg.nope or cfg.ada_rope):
            if self.rope_cache is None or T > self.max_len or self.rope_cache[0].device != idx.device:
                self.max_len = max(T, self.max_len)
                self.rope_cache = self.build_rope_cache(idx, self.max_len)
            rope = (self.rope_cache[0][:T], self.rope_cache[1][:T])
        x = self.transformer.wte(idx)
        if self.scale_embed:
            x = x * math.sqrt(cfg.n_embd)
        if getattr(self, "tp_size", 1) > 1:
            # tensor + sequence parallelism: between blocks each rank carries a 1/tp chunk of the flattened tokens
            from archscale_b200.parallel.tp import token_slice
            self._tp_batch_shape = (B, T)
            x = token_slice(x, self.tp_size, self.tp_rank).contiguous()
        input_embed = x
        kv_cache = gmu_mems = None
        self.lc_gate_hist, self.tokens_per_expert, self.token_indices = [], [], []
        self.aux_loss = 0.0
        self.attn_output_rmsnorms, self.mlp_output_rmsnorms = [], []
        self.attn_outlier_pcts, self.mlp_outlier_pcts = [], []
        self.attn_z_means, self.router_z_means = [], []

        h_pending = None
        blocks = list(self.transformer.h)
        from archscale_b200.models.norms import FusedRMSNorm
        use_deferred = (self.compute_dtype == torch.bfloat16 and self.layer_configurator is None
                        and type(self.transformer.ln_f) is FusedRMSNorm and ops.norm.fused_cols_ok(cfg.n_embd)
                        and all(b._deferred_ok(x, None, residual_dropout) for b in blocks))

        def run(block):
            nonlocal x, kv_cache, gmu_mems, input_embed, h_pending
            if use_deferred:
                x, kv_cache, gmu_mems, input_embed, h_pending = block(
                    x, input_embed, rope, max_seq_length, seq_meta, kv_cache=kv_cache, gmu_mems=gmu_mems,
                    compute_dtype=self.compute_dtype, h_pending=h_pending, deferred=True)
            else:
                x, kv_cache, gmu_mems, input_embed = block(
                    x, input_embed, rope, max_seq_length, seq_meta, lc=self.layer_configurator, kv_cache=kv_cache,
                    gmu_mems=gmu_mems, residual_dropout=residual_dropout, lc_gate_hist=self.lc_gate_hist,
                    compute_dtype=self.compute_dtype)
            if self.collect_stats:
                self.attn_output_rmsnorms.append(block.attn_output_rmsnorm)
                self.mlp_output_rmsnorms.append(block.mlp_output_rmsnorm)
                self.attn_outlier_pcts.append(block.attn_outlier_pct)
                self.mlp_outlier_pcts.append(block.mlp_outlier_pct)
                self.attn_z_means.append(block.attn_z_mean)
                self.router_z_means.append(block.router_z_mean)
            if cfg.moe:
                self.aux_loss = self.aux_loss + block.mlp.aux_loss
                self.token_indices.append(block.mlp.token_indices)
                self.tokens_per_expert.append(block.mlp.tokens_per_expert)

        bc = self.block_cfg
        if bc.share_per_layer > 0:
            reps = bc.n_layer // bc.share_group // bc.share_per_layer
            for g in range(bc.share_group):
                for _ in range(reps):
                    for block in self.transformer.h[g * bc.share_per_layer:(g + 1) * bc.share_per_layer]:
                        run(block)
        else:
            for block in self.transformer.h:
                run(block)
        if cfg.sum_skip:
            x = input_embed
        if use_deferred:
            scale = 1.0 / math.sqrt(2 * cfg.n_layer) if cfg.depth_scale else 1.0
            stream = torch.float32 if cfg.residual_in_fp32 else self.compute_dtype
            _, x = ops.add_rms_norm(x, h_pending, self.transformer.ln_f.weight, self.transformer.ln_f.eps, scale,
                                    self.compute_dtype, stream)
        else:
            x = _norm_to(self.transformer.ln_f, x, self.compute_dtype)
        if self.logit_scale != 1.0:
            x = x * self.logit_scale
        if use_flce_loss:
            return CausalLMOutput(logits=x, weight=self.lm_head.weight)
        return CausalLMOutput(logits=self.lm_head(x).float())
