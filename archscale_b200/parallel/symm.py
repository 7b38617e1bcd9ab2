"""Symmetric heap over CUDA IPC and the peer-memory collectives of the FSDP engine / Muon step.

Every rank of the shard group allocates one block of device memory of the same size and maps every
peer's block (``cudaIpcOpenMemHandle``); objects are placed by a deterministic bump allocator, so an
object has the same offset on every rank and a kernel reaches rank ``p``'s copy at
``bases[p] + offset``.  The kernels (``csrc/comm.cu``) use plain NVLink loads — no NCCL on these
paths, no multicast:

* **all-gather** — the low-precision parameter shards live *in* the heap; gathering unit ``k`` is one
  pull kernel that reads every peer's shard straight into the local gathered buffer.  Shards only
  change in the optimizer step, which ends with a device-side barrier, so gathers need no handshake.
* **reduce-scatter** — the fp32 flat gradient buffers live in the heap (the wgrad GEMMs accumulate
  into them directly); after a unit's backward a rank posts a signal, waits for its peers' signals
  (bounded) and pulls + sums its own slice from all peers in fixed rank order (bitwise reproducible),
  fused with the ``1/world`` scale and the accumulation into the gradient shard.
* **Muon transport** — the pre-orthogonalisation update U (bf16) is gathered with the same pull
  kernel; the orthogonalised O returns with a bf16 pull-reduce.

Replaces the NCCL all-gather / reduce-scatter that torch FSDP2 issues for the reference
(`pretrain.py:536-563`) and the all-to-all pair of its Muon (`lit_gpt/optim/muon.py:531-558`).
"""
from __future__ import annotations

from typing import Dict, Optional, List, Tuple

import torch
import torch.distributed as dist

from archscale_b200.ops import backend

_SIGNAL_BYTES = 1 << 16      # 2048 channels × 8 ranks × 4 bytes
_ALIGN = 1024


class SymmetricHeap:
    def __init__(self, group, nbytes: int, device: torch.device) -> None:
        self.ext = backend.require_extension()
        self.group, self.device = group, device
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        assert self.world <= 8, "peer-memory collectives support up to 8 ranks per group"
        self.nbytes = ((nbytes + _SIGNAL_BYTES + _ALIGN - 1) // _ALIGN) * _ALIGN
        self.base = self.ext.symm_alloc(self.nbytes)
        handles: List[bytes] = [None] * self.world
        dist.all_gather_object(handles, self.ext.symm_ipc_handle(self.base), group=group)
        self.bases = [self.base if r == self.rank else self.ext.symm_ipc_open(handles[r]) for r in range(self.world)]
        self.cursor = _SIGNAL_BYTES
        self.epochs: Dict[int, int] = {}
        dist.barrier(group=group)

    def alloc(self, nbytes: int) -> int:
        off = self.cursor
        self.cursor = ((off + nbytes + _ALIGN - 1) // _ALIGN) * _ALIGN
        assert self.cursor <= self.nbytes, "symmetric heap exhausted"
        return off

    def tensor(self, off: int, shape, dtype: torch.dtype) -> torch.Tensor:
        return self.ext.symm_tensor(self.base + off, list(shape), dtype, self.device.index or 0)

    def next_epoch(self, channel: int) -> int:
        e = self.epochs.get(channel, 0) + 1
        self.epochs[channel] = e
        return e

    def barrier(self, channel: int = 0) -> None:
        self.ext.symm_barrier(self.bases, 0, channel, self.rank, self.next_epoch(channel))

    def post(self, channel: int) -> int:
        e = self.next_epoch(channel)
        self.ext.symm_post(self.bases, 0, channel, self.rank, e)
        return e

    def wait(self, channel: int, epoch: int) -> None:
        self.ext.symm_wait(self.bases, 0, channel, self.rank, epoch)


class SymmetricContext:
    """Places the engine's shards / gradient buffers in a symmetric heap and serves its collectives."""

    def __init__(self, engine, comm_ctas: int = 64, reduce_ctas: int = 296) -> None:
        self.engine = engine
        self.comm_ctas = comm_ctas
        self.reduce_ctas = reduce_ctas      # latency-bound pulls: co-resident with the GEMM CTAs, light on ALUs
        groups = [g for g in engine.groups() if g.world > 1]
        esize = lambda dt: torch.empty((), dtype=dt).element_size()
        need = 0
        for g in groups:
            need += g.shard_numel * esize(g.dtype) + _ALIGN          # low-precision shard
            need += g.padded * 4 + _ALIGN                            # fp32 flat gradients
            need += g.shard_numel * 2 + g.padded * 2 + 2 * _ALIGN    # Muon: U shard, O full (bf16)
        self.heap = SymmetricHeap(engine.group, need, engine.device)
        self.ext = self.heap.ext
        self.meta: Dict[int, dict] = {}
        assert 1 + 4 * len(groups) <= _SIGNAL_BYTES // (8 * 4), \
            f"{len(groups)} flat groups need {1 + 4 * len(groups)} signal channels; the heap has {_SIGNAL_BYTES // 32}"
        for i, g in enumerate(groups):
            # channels of a group: +0 gradients posted, +1 Muon U posted, +2 Muon O posted, +3 gradient slice read
            m = {"chan": 1 + 4 * i, "rd_epoch": None}
            m["lp_off"] = self.heap.alloc(g.shard_numel * esize(g.dtype))
            lp = self.heap.tensor(m["lp_off"], (g.shard_numel,), g.dtype)
            lp.copy_(g.master)
            if g.dtype == torch.float32:
                # fp32 groups gather the master values; keep a heap mirror that refresh_lp() updates
                g.fp32_mirror = lp
            g.shard_lp = lp
            g.lp_stale = False
            m["fg_off"] = self.heap.alloc(g.padded * 4)
            g.symm_full_grad = self.heap.tensor(m["fg_off"], (g.padded,), torch.float32)
            g.symm_fg_dirty = False
            m["u_off"] = self.heap.alloc(g.shard_numel * 2)
            m["u"] = self.heap.tensor(m["u_off"], (g.shard_numel,), torch.bfloat16)
            m["o_off"] = self.heap.alloc(g.padded * 2)
            m["o"] = self.heap.tensor(m["o_off"], (g.padded,), torch.bfloat16)
            self.meta[id(g)] = m
        torch.cuda.synchronize()
        self.step_barrier()

    # ------------------------------------------------------------------ engine hooks
    def lp_shard(self, g) -> torch.Tensor:
        """Refresh (if stale) and return the heap-resident low-precision shard of ``g``."""
        if g.lp_stale:
            g.shard_lp.copy_(g.master)
            g.lp_stale = False
        return g.shard_lp

    def step_barrier(self) -> None:
        """All ranks have finished writing their shards / reading their peers' buffers for this step."""
        self.heap.barrier(0)
        for m in self.meta.values():
            m["rd_epoch"] = None         # nobody still reads a gradient buffer of the finished step

    def wait_readers(self, g) -> None:
        """Before the heap gradient buffer of ``g`` is zeroed or accumulated into again inside one optimizer step
        (gradient accumulation): wait until every peer has pulled its slice of the previous micro-step from it."""
        m = self.meta[id(g)]
        if m["rd_epoch"] is not None:
            self.heap.wait(m["chan"] + 3, m["rd_epoch"])
            m["rd_epoch"] = None
            backend.count_launch()

    def all_gather(self, g, lp: torch.Tensor) -> None:
        m = self.meta[id(g)]
        self.ext.allgather_pull(self.heap.bases, m["lp_off"], g.full, g.shard_numel * g.full.element_size(),
                                self.heap.rank, self.comm_ctas)
        backend.count_launch()

    def ag_gemm(self, x2: torch.Tensor, g, n_out: int, n_copy: int = 16) -> torch.Tensor:
        """``x2 @ Wᵀ`` for the first weight ``W (n_out × K)`` of group ``g`` with the all-gather of the whole
        group fused into the same kernel launch."""
        m = self.meta[id(g)]
        if "ag_flags" not in m:
            n_chunks = (g.padded * g.full.element_size() + 256 * 1024 - 1) // (256 * 1024)
            m["ag_flags"] = torch.zeros(n_chunks, dtype=torch.int32, device=self.engine.device)
            m["ag_epoch"] = 0
        m["ag_epoch"] += 1
        out = self.ext.ag_gemm(x2, self.heap.bases, m["lp_off"], g.full, g.shard_numel * g.full.element_size(), 0,
                               n_out, m["ag_flags"], m["ag_epoch"], self.heap.rank, n_copy)
        backend.count_launch()
        return out

    def reduce_scatter(self, g, out: torch.Tensor, full_grad: torch.Tensor, scale: float) -> None:
        m = self.meta[id(g)]
        assert full_grad.data_ptr() == g.symm_full_grad.data_ptr(), "gradient buffer must live in the symmetric heap"
        e = self.heap.post(m["chan"])
        self.heap.wait(m["chan"], e)
        self.ext.reduce_scatter_pull(self.heap.bases, m["fg_off"], out, self.heap.rank, scale, False, self.reduce_ctas)
        m["rd_epoch"] = self.heap.post(m["chan"] + 3)       # "I have read my slice of everybody's buffer"
        backend.count_launch(4)

    # ------------------------------------------------------------------ Muon transport
    def u_buffer(self, g) -> torch.Tensor:
        return self.meta[id(g)]["u"]

    def o_buffer(self, g) -> torch.Tensor:
        return self.meta[id(g)]["o"]

    def gather_flat(self, g, u_shard: torch.Tensor) -> torch.Tensor:
        m = self.meta[id(g)]
        assert u_shard.data_ptr() == m["u"].data_ptr()
        e = self.heap.post(m["chan"] + 1)
        self.heap.wait(m["chan"] + 1, e)
        full = torch.empty(g.padded, dtype=torch.bfloat16, device=self.engine.device)
        self.ext.allgather_pull(self.heap.bases, m["u_off"], full, g.shard_numel * 2, self.heap.rank, self.comm_ctas)
        backend.count_launch(3)
        return full

    @staticmethod
    def _piece_table(pieces, rank: int, world: int, device) -> Optional[torch.Tensor]:
        """``pieces``: (src_rank, src_elem, dst_elem, n_elem) of bf16 ranges → int64 [n, 3] device table of 16-byte-vector
        pieces of at most 4096 vectors, interleaved over the source ranks starting after ``rank`` (no two ranks start on
        the same peer).  None if a range is not 16-byte aligned."""
        per_rank = [[] for _ in range(world)]
        for src_rank, src, dst, n in pieces:
            if src % 8 or dst % 8 or n % 8:
                return None
            sv, dv, nv = src // 8, dst // 8, n // 8
            while nv > 0:
                step = min(nv, 4096)
                per_rank[(src_rank - rank - 1) % world].append((sv, dv, step | (src_rank << 32)))
                sv, dv, nv = sv + step, dv + step, nv - step
        rows = []
        depth = max((len(l) for l in per_rank), default=0)
        for i in range(depth):
            rows.extend(l[i] for l in per_rank if i < len(l))
        return torch.tensor(rows, dtype=torch.int64, device=device).reshape(-1, 3)

    def gather_owned(self, g, u_shard: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
        """Flat-sized buffer in which only the ranges named by ``table`` (this rank's own matrices) are filled, each
        from the shards that hold it: a rank moves 1/world of what :meth:`gather_flat` moves
        (reference: the all-to-all of `lit_gpt/optim/muon.py:531-535`)."""
        m = self.meta[id(g)]
        assert u_shard.data_ptr() == m["u"].data_ptr()
        e = self.heap.post(m["chan"] + 1)
        self.heap.wait(m["chan"] + 1, e)
        full = torch.empty(g.padded, dtype=torch.bfloat16, device=self.engine.device)
        self.ext.pull_pieces(self.heap.bases, m["u_off"], full, table, self.comm_ctas)
        backend.count_launch(3)
        return full

    def scatter_owned(self, g, o_full: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
        """This rank's shard of the orthogonalised updates, every range copied from the one rank that computed it
        (no sum, so the owners' buffers need no zero fill; reference: `lit_gpt/optim/muon.py:554-558`)."""
        m = self.meta[id(g)]
        assert o_full.data_ptr() == m["o"].data_ptr()
        e = self.heap.post(m["chan"] + 2)
        self.heap.wait(m["chan"] + 2, e)
        out = torch.empty(g.shard_numel, dtype=torch.bfloat16, device=self.engine.device)
        self.ext.pull_pieces(self.heap.bases, m["o_off"], out, table, self.comm_ctas)
        backend.count_launch(3)
        return out

    def scatter_flat(self, g, o_full: torch.Tensor) -> torch.Tensor:
        m = self.meta[id(g)]
        assert o_full.data_ptr() == m["o"].data_ptr()
        e = self.heap.post(m["chan"] + 2)
        self.heap.wait(m["chan"] + 2, e)
        out = torch.empty(g.shard_numel, dtype=torch.bfloat16, device=self.engine.device)
        self.ext.reduce_scatter_pull(self.heap.bases, m["o_off"], out, self.heap.rank, 1.0, False, self.reduce_ctas)
        backend.count_launch(3)
        return out
