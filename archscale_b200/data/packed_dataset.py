"""Packed token shards (``LITPKDS`` ``.bin`` files): writer, sharded reader, weighted mixture,
plus the synthetic token source the benchmarks use.

Format and sampling order follow the reference (`lit_gpt/packed_dataset.py:23-34,50-67,
115-120,157-268`): 24-byte header (magic ``b"LITPKDS"``, ``<Q`` version 1, ``<B`` dtype code,
``<Q`` chunk size) followed by tokens; files are dealt round-robin to (rank, worker) shards,
``n_chunks`` files are mapped at a time and their ``block_size``-token blocks are visited in a
``default_rng(seed)`` permutation; `CombinedDataset` (`:271-300`) draws the source of every
sample with ``random.Random(seed).choices`` and tags samples whose path contains ``msr_code``.

Additions: :meth:`PackedDatasetIterator.skip` fast-forwards in O(files) without reading tokens
(the reference replays and discards batches on resume, `pretrain.py:788-796`), and
:class:`PinnedBatchLoader` stages batches in pinned host memory on a background thread.
"""
from __future__ import annotations

import os
import queue
import random
import struct
import threading
from typing import Iterator, List, Optional, Sequence, Tuple

import numpy as np
import torch

dtypes = {1: np.uint8, 2: np.int8, 3: np.int16, 4: np.int32, 5: np.int64, 6: np.float32, 7: np.float64, 8: np.uint16}
HDR_MAGIC = b"LITPKDS"
HDR_SIZE = 24


def code(dtype) -> int:
    for k, v in dtypes.items():
        if v == dtype:
            return k
    raise ValueError(dtype)


class PackedDatasetBuilder:
    """Accumulates token arrays and writes fixed-size chunks ``{prefix}_{counter:010d}.bin``."""

    def __init__(self, outdir: str, prefix: str, chunk_size: int, sep_token: int, dtype="auto",
                 vocab_size: Optional[int] = None) -> None:
        if dtype == "auto":
            if vocab_size is None:
                raise ValueError("vocab_size is required when dtype='auto'")
            self._dtype = np.uint16 if vocab_size < 65500 else np.int32
        else:
            self._dtype = dtype
        self._outdir, self._prefix, self._chunk_size, self._sep_token = outdir, prefix, chunk_size, sep_token
        self._arr = np.full(chunk_size, sep_token, dtype=self._dtype)
        self._idx = 0
        self._counter = 0
        self._filenames: List[str] = []
        os.makedirs(outdir, exist_ok=True)

    @property
    def dtype(self):
        return self._dtype

    @property
    def filenames(self) -> List[str]:
        return list(self._filenames)

    def _write_chunk(self) -> None:
        path = os.path.join(self._outdir, f"{self._prefix}_{self._counter:010d}.bin")
        with open(path, "wb") as f:
            f.write(HDR_MAGIC)
            f.write(struct.pack("<Q", 1))
            f.write(struct.pack("<B", code(self._dtype)))
            f.write(struct.pack("<Q", self._chunk_size))
            f.write(self._arr.tobytes(order="C"))
        self._filenames.append(path)
        self._counter += 1
        self._arr.fill(self._sep_token)
        self._idx = 0

    def add_array(self, arr: np.ndarray) -> None:
        arr = np.asarray(arr)
        while self._idx + arr.shape[0] > self._chunk_size:
            part = self._chunk_size - self._idx
            self._arr[self._idx:] = arr[:part]
            self._write_chunk()
            arr = arr[part:]
        n = arr.shape[0]
        self._arr[self._idx:self._idx + n] = arr
        self._idx += n

    def write_reminder(self) -> None:
        """Flush the partially filled chunk (padded with the separator token)."""
        self._write_chunk()


def read_header(path: str) -> Tuple[type, int]:
    with open(path, "rb") as f:
        assert f.read(len(HDR_MAGIC)) == HDR_MAGIC, f"{path}: not a packed dataset file"
        (version,) = struct.unpack("<Q", f.read(8))
        assert version == 1
        (dtype_code,) = struct.unpack("<B", f.read(1))
        (chunk_size,) = struct.unpack("<Q", f.read(8))
    return dtypes[dtype_code], chunk_size


class PackedDatasetIterator:
    def __init__(self, filenames: Sequence[str], n_chunks: int, block_size: int, seed: int, shuffle: bool,
                 drop_last: bool = True) -> None:
        self._filenames = list(filenames)
        self._n_chunks, self._block_size = n_chunks, block_size
        self._rng = np.random.default_rng(seed) if shuffle else None
        self._shuffle, self._drop_last = shuffle, drop_last
        self._file_idx = 0
        self._dtype = None
        self._n_blocks = 0
        self._mmaps: List[np.memmap] = []
        self._block_idxs: Sequence[int] = []
        self._curr_idx = 0
        if not self._filenames:
            raise StopIteration
        self._load_n_chunks()

    def _next_group_size(self) -> int:
        n_files = len(self._filenames)
        if self._drop_last:
            if self._n_chunks > n_files - self._file_idx:
                self._file_idx = 0
            return min(self._n_chunks, n_files)
        if self._file_idx == n_files:
            self._file_idx = 0
        remaining = n_files - self._file_idx
        if self._n_chunks > n_files:
            return n_files
        return remaining if 0 < remaining < self._n_chunks else self._n_chunks

    def _load_n_chunks(self, map_files: bool = True) -> None:
        self._mmaps = []
        n = self._next_group_size()
        paths = [self._filenames[self._file_idx + i] for i in range(n)]
        if self._dtype is None:
            self._dtype, chunk = read_header(paths[0])
            self._n_blocks = chunk // self._block_size
        if map_files:
            self._mmaps = [np.memmap(p, mode="r", order="C", offset=HDR_SIZE, dtype=self._dtype) for p in paths]
        self._pending_paths = paths
        self._file_idx += n
        total = n * self._n_blocks
        self._block_idxs = self._rng.permutation(total) if self._shuffle else range(total)
        self._curr_idx = 0

    def skip(self, n_samples: int) -> None:
        """Advance as if ``n_samples`` had been read: same RNG stream, no token IO."""
        while n_samples > 0:
            left = len(self._block_idxs) - self._curr_idx
            if n_samples < left:
                self._curr_idx += n_samples
                break
            n_samples -= left
            self._load_n_chunks(map_files=False)
        if not self._mmaps:
            self._mmaps = [np.memmap(p, mode="r", order="C", offset=HDR_SIZE, dtype=self._dtype)
                           for p in self._pending_paths]

    def __iter__(self):
        return self

    def __next__(self) -> torch.Tensor:
        if self._curr_idx >= len(self._block_idxs):
            self._load_n_chunks()
        block_idx = int(self._block_idxs[self._curr_idx])
        chunk_id, within = divmod(block_idx, self._n_blocks)
        start = within * self._block_size
        arr = self._mmaps[chunk_id][start:start + self._block_size]
        self._curr_idx += 1
        return torch.from_numpy(arr.astype(np.int64))


class PackedDataset(torch.utils.data.IterableDataset):
    def __init__(self, filenames: Sequence[str], n_chunks: int, block_size: int, seed: int = 12345,
                 shuffle: bool = True, drop_last: bool = True, num_processes: int = 1, process_rank: int = 0) -> None:
        self._filenames = list(filenames)
        self._n_chunks, self._block_size, self._seed = n_chunks, block_size, seed
        self._shuffle, self._drop_last = shuffle, drop_last
        self._num_processes, self._process_rank = num_processes, process_rank

    def __iter__(self) -> PackedDatasetIterator:
        info = torch.utils.data.get_worker_info()
        workers, wid = (info.num_workers, info.id) if info is not None else (1, 0)
        shards = workers * self._num_processes
        shard_id = self._process_rank * workers + wid
        usable = len(self._filenames) // shards * shards
        return PackedDatasetIterator(self._filenames[shard_id:usable:shards], self._n_chunks, self._block_size,
                                     self._seed, self._shuffle, self._drop_last)


class CombinedDatasetIterator:
    def __init__(self, datasets: Sequence[PackedDataset], seed: int, weights: Sequence[float]) -> None:
        self._datasets = [(iter(ds), "msr_code" in ds._filenames[0]) for ds in datasets]
        self._weights = list(weights)
        self._rng = random.Random(seed)

    def __iter__(self):
        return self

    def __next__(self):
        idx = self._rng.choices(range(len(self._datasets)), weights=self._weights, k=1)[0]
        it, is_code = self._datasets[idx]
        return next(it), is_code

    def skip(self, n_samples: int) -> None:
        counts = [0] * len(self._datasets)
        for _ in range(n_samples):
            counts[self._rng.choices(range(len(self._datasets)), weights=self._weights, k=1)[0]] += 1
        for (it, _), c in zip(self._datasets, counts):
            if c:
                it.skip(c)


class CombinedDataset(torch.utils.data.IterableDataset):
    def __init__(self, datasets: Sequence[PackedDataset], seed: int, weights: Optional[Sequence[float]] = None) -> None:
        self._seed, self._datasets = seed, list(datasets)
        n = len(self._datasets)
        self._weights = list(weights) if weights is not None else [1 / n] * n

    def __iter__(self) -> CombinedDatasetIterator:
        return CombinedDatasetIterator(self._datasets, self._seed, self._weights)


class SyntheticTokens:
    """Uniform-random token IDs of a fixed shape (seeded per rank): the benchmark data source."""

    def __init__(self, vocab_size: int, block_size: int, seed: int = 0, rank: int = 0,
                 eos_token_id: Optional[int] = None, doc_len_lognormal: Optional[Tuple[float, float]] = None,
                 doc_len_clip: Tuple[int, int] = (64, 8192)) -> None:
        self.vocab_size, self.block_size = vocab_size, block_size
        self._gen = torch.Generator().manual_seed(seed * 1000003 + rank)
        self._np = np.random.default_rng(seed * 1000003 + rank)
        self.eos, self.lognormal, self.clip = eos_token_id, doc_len_lognormal, doc_len_clip

    def __iter__(self):
        return self

    def skip(self, n: int) -> None:
        for _ in range(n):
            next(self)

    def __next__(self):
        lo = 0 if self.eos is None else 3
        x = torch.randint(lo, self.vocab_size, (self.block_size,), generator=self._gen, dtype=torch.int64)
        if self.eos is not None and self.lognormal is not None:
            # documents with lognormal lengths (given mean / sigma of the length itself), packed back to back
            mean, sigma = self.lognormal
            mu = np.log(mean) - 0.5 * sigma * sigma
            pos = 0
            while pos < self.block_size:
                n = int(np.clip(self._np.lognormal(mu, sigma), *self.clip))
                pos += n
                if pos - 1 < self.block_size:
                    x[pos - 1] = self.eos
        return x, False


class PinnedBatchLoader:
    """Collates ``batch_size`` samples into pinned host memory on a background thread and hands
    out ``(tokens_cpu_pinned, is_code)``; the trainer issues the (async) host→device copy."""

    def __init__(self, sample_iter: Iterator, batch_size: int, prefetch: int = 4, pin: Optional[bool] = None) -> None:
        self._it, self._bs = sample_iter, batch_size
        self._pin = torch.cuda.is_available() if pin is None else pin
        self._q: "queue.Queue" = queue.Queue(maxsize=prefetch)
        self._stop = threading.Event()
        self._done = False      # the stream ended (or failed): every later __next__ raises again instead of blocking
        self._thread = threading.Thread(target=self._work, daemon=True)
        self._thread.start()

    def _work(self) -> None:
        try:
            while not self._stop.is_set():
                samples, flags = [], []
                for _ in range(self._bs):
                    s = next(self._it)
                    if isinstance(s, tuple):
                        s, f = s
                    else:
                        f = False
                    samples.append(s)
                    flags.append(f)
                batch = torch.stack(samples)
                if self._pin:
                    batch = batch.pin_memory()
                self._q.put((batch, any(flags)))
        except StopIteration:
            self._q.put(None)
        except BaseException as e:  # noqa: BLE001 - re-raised in the consumer
            self._q.put(e)

    def __iter__(self):
        return self

    def __next__(self):
        if self._done:
            raise StopIteration
        item = self._q.get()
        if item is None:
            self._done = True
            raise StopIteration
        if isinstance(item, BaseException):
            self._done = True
            raise item
        return item

    def close(self) -> None:
        self._stop.set()
        self._done = True
        try:
            while True:
                self._q.get_nowait()
        except queue.Empty:
            pass
