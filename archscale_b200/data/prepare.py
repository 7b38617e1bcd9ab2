"""Tokenise text corpora into packed ``.bin`` chunks (``PackedDatasetBuilder``), one builder per worker process.

One tool for the corpus-specific scripts of the reference (`scripts/prepare_slimpajama.py:30-110`,
`prepare_redpajama.py`, `prepare_starcoder.py`, `tokenize_pretrained.py`): they differ only in the file pattern,
the container (``.jsonl``, ``.jsonl.zst``, ``.parquet``) and the text column.  Chunks hold ``chunk_size`` tokens
(default 2049·1024, i.e. 1024 training rows of 2048+1), documents are separated by the BOS id, and the trailing
partial chunk is dropped (it would be padding only).

    python -m archscale_b200.data.prepare --source_path data/SlimPajama --tokenizer_path ckpt/llama \
        --destination_path data/slim_packed --pattern 'train/chunk*/*.jsonl.zst' --prefix train_slimpajama
    python -m archscale_b200.data.prepare --preset starcoder --source_path data/starcoderdata ...
"""
from __future__ import annotations

import argparse
import glob
import io
import json
import os
import time
from multiprocessing import Process, cpu_count
from typing import Callable, Iterator, List, Optional

import numpy as np

from archscale_b200.data.packed_dataset import PackedDatasetBuilder

PRESETS = {
    "slimpajama": dict(pattern="{split}/chunk*/*.jsonl.zst", text_key="text", prefix="{split}_slimpajama"),
    "redpajama": dict(pattern="*/*.jsonl", text_key="text", prefix="{split}_redpajama"),
    "starcoder": dict(pattern="*/*.parquet", text_key="content", prefix="{split}_starcoder"),
    "parquet": dict(pattern="**/*.parquet", text_key="text", prefix="{split}_parquet"),
}


def iter_texts(path: str, text_key: str) -> Iterator[str]:
    """Yield the documents of one file (``.jsonl``, ``.jsonl.zst`` / ``.zst``, ``.parquet``, ``.txt``)."""
    if path.endswith(".parquet"):
        import pyarrow.parquet as pq
        pf = pq.ParquetFile(path)
        for batch in pf.iter_batches(columns=[text_key]):
            for t in batch.column(0).to_pylist():
                if t:
                    yield t
    elif path.endswith(".zst"):
        import zstandard as zstd
        with open(path, "rb") as raw:
            with io.TextIOWrapper(zstd.ZstdDecompressor().stream_reader(raw), encoding="utf-8") as f:
                for row in f:
                    if row.strip():
                        yield json.loads(row)[text_key]
    elif path.endswith(".txt"):
        with open(path, encoding="utf-8") as f:
            yield f.read()
    else:
        with open(path, encoding="utf-8") as f:
            for row in f:
                if row.strip():
                    yield json.loads(row)[text_key]


def tokenize_files(files: List[str], encode: Callable[[str], "np.ndarray"], sep_token: int, vocab_size: int,
                   destination_path: str, prefix: str, chunk_size: int, text_key: str,
                   keep_remainder: bool = False) -> List[str]:
    builder = PackedDatasetBuilder(outdir=destination_path, prefix=prefix, chunk_size=chunk_size, sep_token=sep_token,
                                   dtype="auto", vocab_size=vocab_size)
    for path in files:
        for text in iter_texts(path, text_key):
            builder.add_array(np.asarray(encode(text), dtype=builder.dtype))
    if keep_remainder:
        builder.write_reminder()
    return builder.filenames


def _worker(files, tokenizer_path, destination_path, prefix, chunk_size, text_key, keep_remainder):
    from archscale_b200.data.tokenizer import Tokenizer
    tok = Tokenizer(tokenizer_path)
    sep = tok.bos_id if tok.bos_id is not None else tok.eos_id
    tokenize_files(files, lambda s: tok.encode(s).numpy(), sep, tok.vocab_size, destination_path, prefix, chunk_size,
                   text_key, keep_remainder)


def prepare(source_path: str, tokenizer_path: str, destination_path: str, pattern: str, prefix: str,
            text_key: str = "text", chunk_size: int = 2049 * 1024, percentage: float = 1.0,
            num_processes: Optional[int] = None, keep_remainder: bool = False) -> None:
    files = sorted(glob.glob(os.path.join(source_path, pattern), recursive=True))
    files = files[:max(int(len(files) * percentage), 1)]
    if not files:
        raise RuntimeError(f"no files match {pattern} under {source_path}")
    n = min(num_processes or cpu_count(), len(files))
    t0 = time.time()
    procs = []
    for i, subset in enumerate(np.array_split(np.array(files, dtype=object), n)):
        p = Process(target=_worker, args=(list(subset), tokenizer_path, destination_path, f"{prefix}_{i}", chunk_size,
                                          text_key, keep_remainder))
        p.start()
        procs.append(p)
    for p in procs:
        p.join()
        if p.exitcode != 0:
            raise RuntimeError(f"tokenisation worker exited with code {p.exitcode}")
    print(f"{len(files)} files → {destination_path} in {time.time() - t0:.1f} s")


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--preset", choices=sorted(PRESETS), default=None)
    ap.add_argument("--source_path", required=True)
    ap.add_argument("--tokenizer_path", required=True)
    ap.add_argument("--destination_path", required=True)
    ap.add_argument("--split", default="train")
    ap.add_argument("--pattern", default=None)
    ap.add_argument("--prefix", default=None)
    ap.add_argument("--text_key", default=None)
    ap.add_argument("--chunk_size", type=int, default=2049 * 1024)
    ap.add_argument("--percentage", type=float, default=1.0)
    ap.add_argument("--num_processes", type=int, default=None)
    ap.add_argument("--keep_remainder", action="store_true")
    a = ap.parse_args()
    ps = PRESETS.get(a.preset or "", {})
    pattern = (a.pattern or ps.get("pattern") or "**/*.jsonl").format(split=a.split)
    prefix = (a.prefix or ps.get("prefix") or "{split}_data").format(split=a.split)
    prepare(a.source_path, a.tokenizer_path, a.destination_path, pattern, prefix, a.text_key or ps.get("text_key", "text"),
            a.chunk_size, a.percentage, a.num_processes, a.keep_remainder)


if __name__ == "__main__":
    main()
