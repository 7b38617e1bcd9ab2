"""Packing helpers for padded batches (`lit_gpt/bert_padding.py`): drop the padded positions of a (B, T, …) batch into
one (total, …) row block with ``cu_seqlens`` and scatter results back.  The attention, conv and scan kernels of this
package take ``cu_seqlens`` / ``seq_idx`` on packed rows directly, so these two functions are all a padded-batch caller
needs around them."""
from __future__ import annotations

from typing import Tuple

import torch
import torch.nn.functional as F


def unpad_input(hidden_states: torch.Tensor, attention_mask: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, int]:
    """hidden_states: (B, T, …); attention_mask: (B, T) with 1 / True for valid tokens.
    Returns (rows (total, …), indices (total,), cu_seqlens (B+1,) int32, max_seqlen)."""
    seqlens = attention_mask.sum(dim=-1, dtype=torch.int32)
    indices = torch.nonzero(attention_mask.flatten(), as_tuple=False).flatten()
    cu_seqlens = F.pad(torch.cumsum(seqlens, dim=0, dtype=torch.int32), (1, 0))
    rows = hidden_states.reshape(-1, *hidden_states.shape[2:]).index_select(0, indices)
    return rows, indices, cu_seqlens, int(seqlens.max()) if seqlens.numel() else 0


def pad_input(rows: torch.Tensor, indices: torch.Tensor, batch: int, seqlen: int) -> torch.Tensor:
    """Inverse of :func:`unpad_input`: (total, …) → (B, T, …) with zeros at the padded positions (differentiable)."""
    out = rows.new_zeros(batch * seqlen, *rows.shape[1:])
    out = out.index_copy(0, indices, rows)
    return out.view(batch, seqlen, *rows.shape[1:])
