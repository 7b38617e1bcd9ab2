"""Token-skipping layer configurator (``_lc`` train-name switch).

Reference: `lit_gpt/layer_configurator.py:33-122`: RMSNorm → depthwise causal conv(4)+SiLU →
2-way softmax gate; tokens with gate > 0.5 are compacted to the front of a shorter sequence
(``compress``), processed by the layer, and scattered back (``extract``).
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from archscale_b200 import ops
from archscale_b200.config import Config
from archscale_b200.models.layers import Linear
from archscale_b200.utils.init import torch_default_init


class LayerConfigurator(nn.Module):
    def __init__(self, config: Config) -> None:
        super().__init__()
        self.norm = config.norm_class(config.n_embd, eps=config.norm_eps)
        self.lc_proj = Linear(config.n_embd, 2, bias=config.bias)
        self.temp = 1.0
        self.conv1d = nn.Conv1d(config.n_embd, config.n_embd, kernel_size=4, groups=config.n_embd, padding=3, bias=False)
        self.index_q = self.gate = self.act_mask = None

    def reset_parameters(self) -> None:
        if hasattr(self.norm, "reset_parameters"):
            self.norm.reset_parameters()
        torch_default_init(self.lc_proj.weight)
        if self.lc_proj.bias is not None:
            nn.init.zeros_(self.lc_proj.bias)
        torch_default_init(self.conv1d.weight)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        ox = x
        h = self.norm(x)
        h = ops.causal_conv1d(h, self.conv1d.weight.squeeze(1), None, activation="silu", channel_last=True)
        gate = F.softmax(self.lc_proj(h).float() / self.temp, dim=-1)[:, :, 1:]
        keep = gate > 0.5                                             # B T 1
        max_q = int(keep.sum(1).max())
        index_q = keep * torch.cumsum(keep.long(), dim=1)              # 0 = dropped, else 1-based slot
        buf = torch.zeros(ox.shape[0], max_q + 1, ox.shape[2], device=ox.device, dtype=torch.float32)
        buf.scatter_(1, index_q.expand(-1, -1, ox.shape[-1]), ox.float())
        self.index_q, self.gate, self.act_mask = index_q, gate, keep
        return buf[:, 1:].to(ox.dtype) if max_q > 0 else (buf * 0).to(ox.dtype)

    def extract(self, h: torch.Tensor) -> torch.Tensor:
        h = F.pad(h, (0, 0, 1, 0))
        return torch.gather(h.float(), -2, self.index_q.expand(-1, -1, h.shape[-1])).type_as(h)
