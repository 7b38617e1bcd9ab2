"""Tokenizer wrapper over SentencePiece (``tokenizer.model``) or Hugging Face tokenizers (``tokenizer.json``).

Same surface as `lit_gpt/tokenizer.py:14-83`: ``bos_id``, ``eos_id``, ``vocab_size``, ``encode(text, bos, eos,
max_length)`` → int32 tensor, ``decode``; ``tokenizer.model`` wins when a folder holds both files.
"""
from __future__ import annotations

import json
import os
from typing import Optional

import torch


class Tokenizer:
    def __init__(self, checkpoint_dir: str) -> None:
        checkpoint_dir = str(checkpoint_dir)
        sp_path = os.path.join(checkpoint_dir, "tokenizer.model")
        hf_path = os.path.join(checkpoint_dir, "tokenizer.json")
        if os.path.isfile(sp_path):
            from sentencepiece import SentencePieceProcessor
            self.processor = SentencePieceProcessor(model_file=sp_path)
            self.backend = "sentencepiece"
            self.bos_id: Optional[int] = self.processor.bos_id()
            self.eos_id: Optional[int] = self.processor.eos_id()
        elif os.path.isfile(hf_path):
            from tokenizers import Tokenizer as HFTokenizer
            self.processor = HFTokenizer.from_file(hf_path)
            self.backend = "huggingface"
            cfg = {}
            cfg_path = os.path.join(checkpoint_dir, "tokenizer_config.json")
            if os.path.isfile(cfg_path):
                with open(cfg_path) as f:
                    cfg = json.load(f)
            tok = lambda t: t["content"] if isinstance(t, dict) else t
            bos, eos = tok(cfg.get("bos_token")), tok(cfg.get("eos_token"))
            self.bos_id = self.token_to_id(bos) if bos is not None else None
            self.eos_id = self.token_to_id(eos) if eos is not None else None
        else:
            raise FileNotFoundError(f"neither tokenizer.model nor tokenizer.json under {checkpoint_dir}")

    @property
    def vocab_size(self) -> int:
        if self.backend == "huggingface":
            return self.processor.get_vocab_size(with_added_tokens=False)
        return self.processor.vocab_size()

    def token_to_id(self, token: str) -> int:
        i = self.processor.token_to_id(token) if self.backend == "huggingface" else self.processor.piece_to_id(token)
        if i is None:
            raise ValueError(f"token {token!r} is not in the vocabulary")
        return i

    def encode(self, string: str, device: Optional[torch.device] = None, bos: bool = False, eos: bool = True,
               max_length: int = -1) -> torch.Tensor:
        ids = self.processor.encode(string).ids if self.backend == "huggingface" else self.processor.encode(string)
        if bos:
            if self.bos_id is None:
                raise NotImplementedError("this tokenizer defines no BOS token")
            ids = [self.bos_id] + ids
        if eos and self.eos_id is not None:
            ids = ids + [self.eos_id]
        if max_length > 0:
            ids = ids[:max_length]
        return torch.tensor(ids, dtype=torch.int, device=device)

    def decode(self, tensor: torch.Tensor) -> str:
        ids = [tensor.item()] if tensor.ndim == 0 else tensor.tolist()
        return self.processor.decode(ids)
