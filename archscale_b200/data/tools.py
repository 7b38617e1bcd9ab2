"""Corpus-side tools around the packed dataset: mixture weights, streaming shuffle, pre-tokenised long-context data,
chat-template extraction and checkpoint / tokenizer download.

Counterparts in the reference: `scripts/reweight_datasets.py` (mixture weights of the leaf folders of a corpus
inventory), `scripts/shuffle_parquet.py` (size-weighted streaming shuffle of many parquet / jsonl files into shards),
`scripts/tokenize_pretrained.py` (text extraction with the chat template, tokenisation of parquet / jsonl trees),
`scripts/prep_prolong_data.py` (re-chunking of pre-tokenised long-context corpora), `scripts/download.py`.
One module with sub-commands:

    python -m archscale_b200.data.tools weights  --data_stats data_stats.txt --output dataset_weights.json --strategy sqrt
    python -m archscale_b200.data.tools shuffle  --input-dir raw/ --output-dir shuffled/ --buffer-rows 200000
    python -m archscale_b200.data.tools tokenize --source_path raw/ --tokenizer_path tok/ --destination_path packed/
    python -m archscale_b200.data.tools rechunk  --source_path prolong/ --destination_path packed64k/ --seq_len 65536
    python -m archscale_b200.data.tools download --repo_id org/name --checkpoint_dir checkpoints
"""
from __future__ import annotations

import argparse
import glob
import json
import math
import os
import random
from typing import Dict, Iterable, Iterator, List, Optional, Sequence, Tuple

import numpy as np

TEXT_KEYS = ("text", "file_contents", "content", "file_content")      # first match wins
ROLE_PREFIX = {"system": "<|system|>", "user": "<|user|>", "assistant": "<|assistant|>"}


# ------------------------------------------------------------------ mixture weights
def parse_token_count(s: str) -> float:
    """'1.79B' / '18.8M' / '3K' / '1234' → number of tokens."""
    s = s.strip()
    mult = {"B": 1e9, "M": 1e6, "K": 1e3}.get(s[-1:].upper())
    return float(s[:-1]) * mult if mult else float(s)


def parse_inventory(path: str, n_levels: int = 6) -> List[Tuple[str, float]]:
    """Tab-separated corpus inventory: a header line, then ``n_levels`` folder-level columns and a token-count column.
    Returns (folder path, tokens) for every row."""
    out = []
    with open(path) as f:
        for line in f.readlines()[1:]:
            parts = line.rstrip("\n").split("\t")
            if len(parts) <= n_levels:
                continue
            levels = [p.strip() for p in parts[:n_levels] if p.strip()]
            if not levels:
                continue
            try:
                out.append(("/".join(levels), parse_token_count(parts[n_levels])))
            except ValueError:
                continue
    return out


def leaf_folders(entries: Sequence[Tuple[str, float]]) -> Dict[str, float]:
    """Folders of the inventory that have no child folder (inner nodes repeat their children's tokens)."""
    paths = sorted({p for p, _ in entries})
    leaves = {}
    for i, p in enumerate(paths):
        nxt = paths[i + 1] if i + 1 < len(paths) else ""
        has_child = nxt.startswith(p + "/") or any(q.startswith(p + "/") for q in paths[i + 1:i + 8])
        if not has_child:
            leaves[p] = dict(entries)[p]
    return leaves


def mixture_weights(tokens: Dict[str, float], strategy: str = "proportional", suffix: str = "") -> Dict[str, float]:
    """Sampling weights (summing to 1) from token counts: proportional, sqrt, log(1 + n) or uniform."""
    f = {"proportional": lambda n: n, "sqrt": math.sqrt, "log": lambda n: math.log(n + 1), "uniform": lambda n: 1.0}
    if strategy not in f:
        raise ValueError(f"unknown weighting strategy {strategy!r}")
    raw = {k: f[strategy](v) for k, v in tokens.items()}
    z = sum(raw.values())
    return {k + suffix: v / z for k, v in raw.items()}


# ------------------------------------------------------------------ text extraction
def apply_chat_template(messages: Iterable[Dict[str, str]]) -> str:
    parts = []
    for m in messages:
        if m["role"] not in ROLE_PREFIX:
            raise ValueError(f"unknown role {m['role']!r}")
        parts.append(f"{ROLE_PREFIX[m['role']]}\n{m['content']}<|end|>\n")
    return "".join(parts)


def extract_text(obj: Dict) -> Optional[str]:
    """Document text of one record: the first known text column, else a ``messages`` list through the chat template."""
    for k in TEXT_KEYS:
        if k in obj:
            return obj[k]
    if "messages" in obj:
        return apply_chat_template(obj["messages"])
    return None


def iter_records(path: str) -> Iterator[Dict]:
    if path.endswith(".parquet"):
        import pyarrow.parquet as pq
        for batch in pq.ParquetFile(path).iter_batches():
            yield from batch.to_pylist()
    else:
        with open(path, encoding="utf-8") as f:
            for ln, line in enumerate(f):
                if line.strip():
                    try:
                        yield json.loads(line)
                    except json.JSONDecodeError as e:
                        print(f"{path}:{ln + 1}: {e}")


def tokenize_tree(source_path: str, tokenizer_path: str, destination_path: str, chunk_size: int = 2049 * 8192,
                  file_types: Sequence[str] = ("*.parquet", "*.jsonl"), nproc: Optional[int] = None, seed: int = 43) -> None:
    """Tokenise every parquet / jsonl file under ``source_path`` (text column or chat messages) into packed chunks."""
    from multiprocessing import Process, cpu_count
    files = sorted(f for t in file_types for f in glob.glob(os.path.join(source_path, "**", t), recursive=True))
    if not files:
        raise RuntimeError(f"no {list(file_types)} under {source_path}")
    random.Random(seed).shuffle(files)
    n = min(nproc or cpu_count(), len(files))
    procs = [Process(target=_tokenize_worker, args=(list(sub), tokenizer_path, destination_path, chunk_size, i))
             for i, sub in enumerate(np.array_split(np.array(files, dtype=object), n)) if len(sub)]
    for p in procs:
        p.start()
    for p in procs:
        p.join()
        if p.exitcode != 0:
            raise RuntimeError(f"tokenisation worker exited with code {p.exitcode}")


def _tokenize_worker(files: List[str], tokenizer_path: str, destination_path: str, chunk_size: int, pid: int) -> None:
    from archscale_b200.data.packed_dataset import PackedDatasetBuilder
    from archscale_b200.data.tokenizer import Tokenizer
    tok = Tokenizer(tokenizer_path)
    sep = tok.bos_id if tok.bos_id is not None else tok.eos_id
    b = PackedDatasetBuilder(outdir=destination_path, prefix=f"train_{pid}", chunk_size=chunk_size, sep_token=sep, dtype="auto",
                             vocab_size=tok.vocab_size)
    for path in files:
        for rec in iter_records(path):
            text = extract_text(rec)
            if text:
                b.add_array(np.asarray(tok.encode(text).numpy(), dtype=b.dtype))


# ------------------------------------------------------------------ streaming shuffle
def build_alias(weights: Sequence[float]) -> Tuple[List[float], List[int]]:
    """Walker alias tables for O(1) sampling proportional to ``weights`` (zeros allowed, not all zero)."""
    n = len(weights)
    z = float(sum(weights))
    scaled = [w * n / z for w in weights]
    prob, alias = [0.0] * n, [0] * n
    small = [i for i, s in enumerate(scaled) if s < 1.0]
    large = [i for i, s in enumerate(scaled) if s >= 1.0]
    while small and large:
        s, l = small.pop(), large.pop()
        prob[s], alias[s] = scaled[s], l
        scaled[l] -= 1.0 - scaled[s]
        (small if scaled[l] < 1.0 else large).append(l)
    for i in small + large:
        prob[i], alias[i] = 1.0, i
    return prob, alias


def sample_alias(prob: Sequence[float], alias: Sequence[int], rng: random.Random) -> int:
    i = rng.randrange(len(prob))
    return i if rng.random() < prob[i] else alias[i]


def _count_rows(path: str) -> int:
    if path.endswith(".parquet"):
        import pyarrow.parquet as pq
        return pq.ParquetFile(path).metadata.num_rows
    with open(path, "rb") as f:
        return sum(1 for line in f if line.strip())


def _batches(path: str, batch_size: int) -> Iterator[List[Dict]]:
    buf = []
    for rec in iter_records(path):
        text = extract_text(rec)
        if text is None:
            continue
        buf.append({"text": text})
        if len(buf) == batch_size:
            yield buf
            buf = []
    if buf:
        yield buf


def shuffle_corpus(input_dir: str, output_dir: str, batch_size: int = 256, buffer_rows: int = 200_000, seed: int = 42,
                   start_idx: Optional[int] = None, end_idx: Optional[int] = None) -> int:
    """Streaming shuffle of the parquet / jsonl files under ``input_dir`` into jsonl shards of about ``buffer_rows`` rows.

    Batches are drawn from the input files with probability proportional to the rows each still holds (alias tables,
    rebuilt when a file runs out), collected in a buffer, permuted and written — documents of different files interleave
    without more than one buffer in memory.  ``start_idx`` / ``end_idx`` restrict the (seed-shuffled) file list so that
    several jobs can share a corpus.  Returns the number of shards written."""
    rng = random.Random(seed)
    files = sorted(glob.glob(os.path.join(input_dir, "**", "*.parquet"), recursive=True)) + \
        sorted(glob.glob(os.path.join(input_dir, "**", "*.jsonl"), recursive=True))
    if not files:
        raise FileNotFoundError(f"no *.parquet / *.jsonl under {input_dir}")
    rng.shuffle(files)
    lo = max(start_idx or 0, 0)
    hi = end_idx if end_idx is not None else (lo + 256 if start_idx is not None else len(files) - 1)
    files = files[lo:hi + 1]
    os.makedirs(output_dir, exist_ok=True)
    remaining = [_count_rows(f) for f in files]
    readers = [_batches(f, batch_size) for f in files]
    tag = f"{lo}_{hi}_" if start_idx is not None else ""
    buf: List[Dict] = []
    shard = 0

    def flush() -> None:
        nonlocal shard, buf
        rng.shuffle(buf)
        with open(os.path.join(output_dir, f"shuffled_{tag}{shard:06d}.jsonl"), "w", encoding="utf-8") as f:
            for rec in buf:
                f.write(json.dumps(rec, ensure_ascii=False) + "\n")
        shard += 1
        buf = []

    while any(remaining):
        prob, alias = build_alias(remaining)
        while True:
            i = sample_alias(prob, alias, rng)
            if remaining[i] == 0:
                continue
            try:
                batch = next(readers[i])
            except StopIteration:
                remaining[i] = 0
                break
            buf.extend(batch)
            remaining[i] = max(remaining[i] - len(batch), 0)
            if len(buf) >= buffer_rows:
                flush()
            if remaining[i] == 0:
                break
    if buf:
        flush()
    return shard


# ------------------------------------------------------------------ pre-tokenised long-context corpora
def rechunk_tokenized(source_path: str, destination_path: str, seq_len: int, rows_per_chunk: int = 128, prefix: str = "train",
                      sep_token: int = 1, vocab_size: int = 32000, pattern: str = "**/*.npy") -> List[str]:
    """Pre-tokenised documents (``.npy`` / ``.bin`` arrays of token ids, one or many documents each) → packed chunks of
    ``rows_per_chunk`` rows of ``seq_len + 1`` tokens, for long-context continuation runs."""
    from archscale_b200.data.packed_dataset import PackedDatasetBuilder
    files = sorted(glob.glob(os.path.join(source_path, pattern), recursive=True))
    if not files:
        raise RuntimeError(f"no files match {pattern} under {source_path}")
    b = PackedDatasetBuilder(outdir=destination_path, prefix=prefix, chunk_size=(seq_len + 1) * rows_per_chunk, sep_token=sep_token,
                             dtype="auto", vocab_size=vocab_size)
    for path in files:
        arr = np.load(path, mmap_mode="r") if path.endswith(".npy") else np.memmap(path, dtype=np.uint16, mode="r")
        b.add_array(np.asarray(arr).reshape(-1).astype(b.dtype))
    return b.filenames


# ------------------------------------------------------------------ download
def download_from_hub(repo_id: str, checkpoint_dir: str = "checkpoints", tokenizer_only: bool = False,
                      from_safetensors: bool = False, access_token: Optional[str] = None) -> str:
    """Fetch tokenizer (and weight) files of a Hugging Face repository; ``.safetensors`` are turned into ``.bin`` files
    that :mod:`archscale_b200.convert` reads.  Needs ``huggingface_hub`` and a network connection."""
    import torch
    from huggingface_hub import snapshot_download
    patterns = ["tokenizer*", "generation_config.json", "config.json"]
    if not tokenizer_only:
        patterns.append("*.safetensors" if from_safetensors else "*.bin*")
    elif from_safetensors:
        raise ValueError("--from_safetensors has no effect with --tokenizer_only")
    directory = os.path.join(checkpoint_dir, repo_id)
    snapshot_download(repo_id, local_dir=directory, allow_patterns=patterns, token=access_token or os.getenv("HF_TOKEN"))
    if from_safetensors:
        from safetensors.torch import load_file
        for st in glob.glob(os.path.join(directory, "*.safetensors")):
            torch.save(load_file(st), st[:-len(".safetensors")] + ".bin")
            os.remove(st)
    return directory


def main(argv: Optional[List[str]] = None) -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="cmd", required=True)
    w = sub.add_parser("weights")
    w.add_argument("--data_stats", default="data_stats.txt")
    w.add_argument("--output", default="dataset_weights.json")
    w.add_argument("--strategy", choices=["proportional", "sqrt", "log", "uniform"], default="proportional")
    w.add_argument("--suffix", default="", help="appended to every folder key (the directory that holds the .bin files)")
    s = sub.add_parser("shuffle")
    s.add_argument("--input-dir", required=True)
    s.add_argument("--output-dir", required=True)
    s.add_argument("--batch-size", type=int, default=256)
    s.add_argument("--buffer-rows", type=int, default=200_000)
    s.add_argument("--seed", type=int, default=42)
    s.add_argument("--start-idx", type=int, default=None)
    s.add_argument("--end-idx", type=int, default=None)
    t = sub.add_parser("tokenize")
    t.add_argument("--source_path", required=True)
    t.add_argument("--tokenizer_path", required=True)
    t.add_argument("--destination_path", required=True)
    t.add_argument("--chunk_size", type=int, default=2049 * 8192)
    t.add_argument("--nproc", type=int, default=None)
    r = sub.add_parser("rechunk")
    r.add_argument("--source_path", required=True)
    r.add_argument("--destination_path", required=True)
    r.add_argument("--seq_len", type=int, required=True)
    r.add_argument("--rows_per_chunk", type=int, default=128)
    r.add_argument("--pattern", default="**/*.npy")
    d = sub.add_parser("download")
    d.add_argument("--repo_id", required=True)
    d.add_argument("--checkpoint_dir", default="checkpoints")
    d.add_argument("--tokenizer_only", action="store_true")
    d.add_argument("--from_safetensors", action="store_true")
    a = ap.parse_args(argv)
    if a.cmd == "weights":
        weights = mixture_weights(leaf_folders(parse_inventory(a.data_stats)), a.strategy, a.suffix)
        with open(a.output, "w") as f:
            json.dump(weights, f, indent=2, sort_keys=True)
        print(f"{len(weights)} leaf datasets → {a.output}")
    elif a.cmd == "shuffle":
        n = shuffle_corpus(a.input_dir, a.output_dir, a.batch_size, a.buffer_rows, a.seed, a.start_idx, a.end_idx)
        print(f"{n} shard(s) written to {a.output_dir}")
    elif a.cmd == "tokenize":
        tokenize_tree(a.source_path, a.tokenizer_path, a.destination_path, a.chunk_size, nproc=a.nproc)
    elif a.cmd == "rechunk":
        print(len(rechunk_tokenized(a.source_path, a.destination_path, a.seq_len, a.rows_per_chunk, pattern=a.pattern)), "chunks")
    else:
        print(download_from_hub(a.repo_id, a.checkpoint_dir, a.tokenizer_only, a.from_safetensors))


if __name__ == "__main__":
    main()
