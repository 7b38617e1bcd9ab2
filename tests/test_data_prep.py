"""Data preparation: jsonl / parquet documents → packed chunks that PackedDataset reads back."""
import json
import os

import numpy as np

from archscale_b200.data import prepare as prep
from archscale_b200.data.packed_dataset import PackedDataset


def test_tokenize_files_round_trip(tmp_path):
    src = tmp_path / "src"
    src.mkdir()
    docs = [f"doc {i} " + "x" * (i % 7) for i in range(40)]
    with open(src / "a.jsonl", "w") as f:
        for d in docs[:20]:
            f.write(json.dumps({"text": d}) + "\n")
    import pyarrow as pa
    import pyarrow.parquet as pq
    pq.write_table(pa.table({"text": docs[20:]}), src / "b.parquet")
    encode = lambda s: np.frombuffer(s.encode(), dtype=np.uint8).astype(np.int64) + 3     # byte-level "tokenizer"
    files = prep.tokenize_files([str(src / "a.jsonl"), str(src / "b.parquet")], encode, sep_token=1, vocab_size=300,
                                destination_path=str(tmp_path / "out"), prefix="train_x", chunk_size=65, text_key="text",
                                keep_remainder=True)
    assert files and all(os.path.getsize(p) == 24 + 65 * 2 for p in files)
    ds = PackedDataset(files, n_chunks=1, block_size=13, shuffle=False, seed=0, num_processes=1, process_rank=0)
    import itertools
    # the iterator wraps around for ever: take exactly one pass, 5 rows of 13 tokens per 65-token chunk
    stream = np.concatenate([np.asarray(x) for x in itertools.islice(iter(ds), 5 * len(files))])
    want = np.concatenate([encode(d) for d in docs])
    assert np.array_equal(stream[:len(want)], want[:len(stream)][:len(want)])
    assert (stream[len(want):] == 1).all()
