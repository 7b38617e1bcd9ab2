"""Phonebook retrieval probe (`eval_phonebook.py:27-140`): a prompt lists ``name: number`` entries, shows two
of them again as few-shot examples and asks for the number of a third; accuracy is exact string match of the
generated number, swept over phonebook lengths.

Names come from a built-in syllable generator (the ``names`` package of the reference is not a dependency), so
prompts are reproducible from the seed alone.

    python -m archscale_b200.eval.phonebook --checkpoint_path ckpt.pth --config sambay_d16 --tokenizer_path tok_dir
"""
from __future__ import annotations

import argparse
import json
import random
from typing import Dict, List, Tuple

import numpy as np
import torch

_SYL = ["an", "bel", "cor", "dan", "el", "fa", "gar", "hol", "is", "jo", "ka", "lin", "mar", "ne", "ol", "pe", "qui", "ro",
        "sa", "ti", "ul", "vi", "wen", "xa", "yo", "zen"]


def _name(rng: random.Random) -> str:
    word = lambda: "".join(rng.choice(_SYL) for _ in range(rng.randint(2, 3))).capitalize()
    return f"{word()} {word()}"


def _phone(rng: random.Random) -> str:
    return str(rng.randint(6, 9)) + "".join(str(rng.randint(0, 9)) for _ in range(9))


def make_example(length: int, rng: random.Random, verbose: bool = False) -> Tuple[str, str]:
    entries = [f"{_name(rng)}: {_phone(rng)}" for _ in range(length)]
    i0, i1, iq = rng.sample(range(length), 3)
    question = entries[iq].split(":")[0] + ":"
    prompt = "\n".join(entries) + "\n\n" + entries[i0] + "\n" + entries[i1] + "\n\n"
    if verbose:
        prompt = "Please find the number of " + question[:-1] + ".\n" + prompt
    return prompt + question, entries[iq].split(":")[1].strip()


def make_batch(length: int, batch_size: int, seed: int, verbose: bool = False) -> Dict[str, List[str]]:
    rng = random.Random(seed)
    pairs = [make_example(length, rng, verbose) for _ in range(batch_size)]
    return {"input": [p for p, _ in pairs], "label": [l for _, l in pairs]}


@torch.no_grad()
def evaluate(wrapper, encode, decode, lengths, batch_size: int = 8, num_batches: int = 1, seed: int = 42,
             max_new_tokens: int = 16, pad_id: int = 0) -> List[Dict[str, float]]:
    """``encode(str) -> list[int]``, ``decode(list[int]) -> str``; prompts are left-padded to a common length."""
    results = []
    for length in lengths:
        hits = total = 0
        for b in range(num_batches):
            batch = make_batch(int(length), batch_size, seed=hash((seed, b, int(length))) & 0xffffffff)
            ids = [encode(p) for p in batch["input"]]
            width = max(len(x) for x in ids)
            inp = torch.full((len(ids), width), pad_id, dtype=torch.long)
            mask = torch.zeros_like(inp)
            for r, x in enumerate(ids):
                inp[r, width - len(x):] = torch.tensor(x)
                mask[r, width - len(x):] = 1
            out = wrapper.generate(inp.to(wrapper.device), attention_mask=mask.to(wrapper.device),
                                   max_length=width + max_new_tokens, return_dict_in_generate=False)
            for r, label in enumerate(batch["label"]):
                text = decode(out[r, width:].tolist())
                hits += int(text.strip().startswith(label))
                total += 1
        results.append({"length": int(length), "accuracy": hits / max(total, 1)})
    return results


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--checkpoint_path", required=True)
    ap.add_argument("--config", required=True)
    ap.add_argument("--tokenizer_path", required=True)
    ap.add_argument("--min_eval_len", type=int, default=20)
    ap.add_argument("--max_eval_len", type=int, default=2048)
    ap.add_argument("--num_eval", type=int, default=100)
    ap.add_argument("--eval_batch_size", type=int, default=32)
    ap.add_argument("--eval_num_batches", type=int, default=3)
    ap.add_argument("--seed", type=int, default=42)
    a = ap.parse_args()
    from archscale_b200.data.tokenizer import Tokenizer
    from archscale_b200.eval.common import load_model
    tok = Tokenizer(a.tokenizer_path)
    wrapper = load_model(a.checkpoint_path, a.config)
    step = (a.max_eval_len + 1 - a.min_eval_len + a.num_eval - 1) // a.num_eval
    lengths = np.arange(a.min_eval_len, a.max_eval_len + 1, step)
    res = evaluate(wrapper, lambda s: tok.encode(s, eos=False).tolist(), lambda ids: tok.decode(torch.tensor(ids)), lengths,
                   a.eval_batch_size, a.eval_num_batches, a.seed, pad_id=tok.eos_id or 0)
    print(json.dumps(res))


if __name__ == "__main__":
    main()
