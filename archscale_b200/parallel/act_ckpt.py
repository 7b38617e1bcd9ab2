"""Activation checkpointing per Block (``--act_ckpt`` / ``--fsdp_save_mem``).

Reference: composable ``checkpoint(module)`` per Block at `pretrain.py:550-555`.  Here the
Block's ``forward`` is wrapped with non-reentrant :func:`torch.utils.checkpoint.checkpoint`;
the FSDP engine keeps parameters gathered while a Block is recomputed inside backward.
"""
from __future__ import annotations

import functools

import torch
from torch.utils.checkpoint import checkpoint


def apply_activation_checkpointing(model: torch.nn.Module, block_cls=None) -> int:
    from archscale_b200.models.gpt import Block
    block_cls = block_cls or Block
    n = 0
    for mod in model.modules():
        if isinstance(mod, block_cls) and not getattr(mod, "_act_ckpt", False):
            inner = mod.forward

            @functools.wraps(inner)
            def wrapped(*args, _inner=inner, **kwargs):
                if not torch.is_grad_enabled():
                    return _inner(*args, **kwargs)
                return checkpoint(_inner, *args, use_reentrant=False, **kwargs)

            mod.forward = wrapped
            mod._act_ckpt = True
            n += 1
    return n
