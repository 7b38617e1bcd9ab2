"""Parameter classification shared by the sharding engine and the optimizers.

Reference rule (`pretrain.py:80,565-592`): a parameter is a *vector* (AdamW group, no weight decay
under μP++) when its name has no ``"weight"`` or contains one of ``conv1d wte lm_head norm ln
layernorm``; everything else is a *matrix* (Muon group).
"""
from __future__ import annotations

VECTOR_NAMES = ("conv1d", "wte", "lm_head", "norm", "ln", "layernorm")


def is_vector_param(name: str) -> bool:
    n = name.lower()
    return ("weight" not in n) or any(v in n for v in VECTOR_NAMES)


def is_matrix_param(name: str, ndim: int) -> bool:
    return ndim >= 2 and not is_vector_param(name)
