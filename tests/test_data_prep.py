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


def test_mixture_weights_from_inventory(tmp_path):
    from archscale_b200.data import tools
    inv = tmp_path / "data_stats.txt"
    rows = ["L1\tL2\tL3\tL4\tL5\tL6\ttokens\tfiles",
            "web\t\t\t\t\t\t3B\t10", "web\tcc\t\t\t\t\t2B\t6", "web\twiki\t\t\t\t\t1B\t4", "code\t\t\t\t\t\t500M\t2"]
    inv.write_text("\n".join(rows) + "\n")
    leaves = tools.leaf_folders(tools.parse_inventory(str(inv)))
    assert leaves == {"web/cc": 2e9, "web/wiki": 1e9, "code": 5e8}        # "web" is an inner node
    w = tools.mixture_weights(leaves, "proportional", suffix="/packed")
    assert abs(sum(w.values()) - 1) < 1e-12 and abs(w["web/cc/packed"] - 2 / 3.5) < 1e-12
    ws = tools.mixture_weights(leaves, "sqrt")
    assert ws["code"] > w["code/packed"]                                   # sqrt flattens the mixture
    assert set(tools.mixture_weights(leaves, "uniform").values()) == {1 / 3}


def test_streaming_shuffle_and_chat_template(tmp_path):
    import json
    from archscale_b200.data import tools
    src = tmp_path / "raw"
    src.mkdir()
    for f in range(3):
        with open(src / f"part{f}.jsonl", "w") as fh:
            for i in range(40):
                fh.write(json.dumps({"text": f"doc {f}-{i}"}) + "\n")
    with open(src / "chat.jsonl", "w") as fh:
        fh.write(json.dumps({"messages": [{"role": "user", "content": "hi"}, {"role": "assistant", "content": "yo"}]}) + "\n")
    n = tools.shuffle_corpus(str(src), str(tmp_path / "out"), batch_size=4, buffer_rows=50, seed=0)
    docs = []
    for p in sorted((tmp_path / "out").glob("*.jsonl")):
        docs += [json.loads(l)["text"] for l in open(p)]
    assert n == len(list((tmp_path / "out").glob("*.jsonl"))) >= 2
    assert sorted(docs) == sorted([f"doc {f}-{i}" for f in range(3) for i in range(40)] + ["<|user|>\nhi<|end|>\n<|assistant|>\nyo<|end|>\n"])
    first = docs[:40]
    assert len({d.split()[1].split("-")[0] for d in first if d.startswith("doc")}) > 1     # files interleave
    prob, alias = tools.build_alias([3, 0, 1])
    import random
    rng = random.Random(0)
    draws = [tools.sample_alias(prob, alias, rng) for _ in range(4000)]
    assert draws.count(1) == 0 and 0.70 < draws.count(0) / 4000 < 0.80
