"""Long-context perplexity over a flat token file (ProofPile protocol of `eval_proofpile.py:50-161`).

The token stream (``uint16`` memmap) is cut into windows of ``seq_length`` tokens that start every
``sliding_window`` tokens; each window is scored with the fused linear-cross-entropy loss (no logits are
materialised), and the mean loss / perplexity over windows is reported.

    python -m archscale_b200.eval.proofpile --checkpoint_path ckpt.pth --config sambay_d16 \
        --data_path test_sampled_data.bin --seq_length 32768 --sliding_window 256 --batch_size 4
"""
from __future__ import annotations

import argparse
import json
import math
from typing import Dict, Iterator

import numpy as np
import torch

from archscale_b200.ops.cross_entropy import FusedLinearCrossEntropyLoss


def iter_windows(tokens: np.ndarray, seq_length: int, batch_size: int, sliding_window: int) -> Iterator[torch.Tensor]:
    starts = list(range(0, max(len(tokens) - seq_length, 0) + 1, sliding_window))
    for i in range(0, len(starts), batch_size):
        rows = [np.asarray(tokens[s:s + seq_length], dtype=np.int64) for s in starts[i:i + batch_size]]
        yield torch.from_numpy(np.stack(rows))


@torch.no_grad()
def evaluate(model, tokens: np.ndarray, seq_length: int, batch_size: int = 1, sliding_window: int = 256,
             device="cuda", max_windows: int = 0) -> Dict[str, float]:
    loss_fn = FusedLinearCrossEntropyLoss()
    losses = []
    seen = 0
    for batch in iter_windows(tokens, seq_length, batch_size, sliding_window):
        ids = batch.to(device)
        out = model(ids, use_flce_loss=True)
        hidden, weight = out.logits, out.weight
        loss = loss_fn(hidden[:, :-1].reshape(-1, hidden.shape[-1]), weight, ids[:, 1:].reshape(-1))
        losses.append(float(loss))
        seen += ids.shape[0]
        if max_windows and seen >= max_windows:
            break
    mean = float(np.mean(losses)) if losses else float("nan")
    return {"loss": mean, "ppl": math.exp(mean) if losses else float("nan"), "windows": seen}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--checkpoint_path", required=True)
    ap.add_argument("--config", required=True)
    ap.add_argument("--data_path", default="test_sampled_data.bin")
    ap.add_argument("--seq_length", type=int, default=32768)
    ap.add_argument("--sliding_window", type=int, default=256)
    ap.add_argument("--batch_size", type=int, default=1)
    ap.add_argument("--max_windows", type=int, default=0)
    a = ap.parse_args()
    from archscale_b200.eval.common import load_model
    wrapper = load_model(a.checkpoint_path, a.config)
    tokens = np.memmap(a.data_path, dtype=np.uint16, mode="r")
    print(json.dumps(evaluate(wrapper.model, tokens, a.seq_length, a.batch_size, a.sliding_window,
                              max_windows=a.max_windows)))


if __name__ == "__main__":
    main()
