"""Expert parallelism: experts sharded over the ``ep`` group, tokens travel to their experts and back.

The reference has no expert parallelism (``ep_degree = 1``, `lit_gpt/moe.py:248-250`); its
``generate_permute_indices`` (`lit_gpt/moe_utils.py:198-271`) only anticipates the (rank × expert)
layout.  Here rank ``r`` of the group owns routed experts ``[r·E_l, (r+1)·E_l)``:

    route (local tokens, all experts) ─► dispatch rows to expert owners ─► grouped expert FFN
                                     ◄─ combine: rows return to their source rank, weighted sum over k

Two transports with identical math:

* ``torch.distributed.all_to_all_single`` with split sizes exchanged first (works on NCCL and on gloo
  CPU ranks; needs one device→host read of the counts per layer) — the baseline;
* peer-memory pulls over the symmetric heap (:class:`PeerDispatcher`): every rank publishes its
  expert-sorted send buffer and per-expert counts in the heap, expert owners pull the contiguous row
  segments that belong to them with bulk NVLink reads (no host synchronisation, no NCCL), results are
  pulled back the same way.

Expert parameters carry ``_ep_local = True``: the FSDP engine never gathers or reduces them (every
rank owns its experts outright); their gradients are complete after the combine-backward.
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist

from archscale_b200 import ops
from archscale_b200.ops import backend
from archscale_b200.ops.gemm import fused_swiglu_enabled


# ------------------------------------------------------------------ setup
def attach(model: torch.nn.Module, mesh, seed: int = 3407) -> None:
    """Bind MoE layers to the expert-parallel group and give every global expert its own init stream."""
    from archscale_b200.models.moe import SonicMoE
    from archscale_b200.utils.init import torch_default_init
    for layer_idx, mod in enumerate(m for m in model.modules() if isinstance(m, SonicMoE)):
        if mod.ep_size <= 1:
            continue
        mod.ep_group = mesh.ep_group
        mod.ep_rank = mesh.ep_rank
        for holder in (mod.mods_in, mod.mods_out):
            holder.weight._ep_local = True
            if holder.bias is not None:
                holder.bias._ep_local = True
            with torch.no_grad():
                # each GLOBAL expert draws from its own seed with the package's default weight init (kaiming-uniform unless
                # --ortho_init / --diag_init / --maxfan_init changed it), as the reference initialises every expert matrix
                # (`lit_gpt/moe.py:533-581`); the values do not depend on the expert-parallel degree
                for e_l in range(mod.n_local):
                    e = mesh.ep_rank * mod.n_local + e_l
                    w = torch.empty(holder.weight.shape[1:], dtype=torch.float32)
                    with torch.random.fork_rng(devices=[]):
                        torch.manual_seed(seed + 1000003 * layer_idx + 7919 * e + (0 if holder is mod.mods_in else 1))
                        torch_default_init(w)
                    holder.weight[e_l].copy_(w.to(holder.weight.dtype))


# ------------------------------------------------------------------ baseline transport (all_to_all)
class _AllToAllRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, out_splits, in_splits, group):
        ctx.group, ctx.out_splits, ctx.in_splits = group, out_splits, in_splits
        out = x.new_empty((sum(out_splits),) + tuple(x.shape[1:]))
        dist.all_to_all_single(out, x.contiguous(), out_splits, in_splits, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        out = g.new_empty((sum(ctx.in_splits),) + tuple(g.shape[1:]))
        dist.all_to_all_single(out, g.contiguous(), ctx.in_splits, ctx.out_splits, group=ctx.group)
        return out, None, None, None


def _moe_ffn_all_to_all(h, w_in, w_out, scores, indices, n_experts: int, group) -> torch.Tensor:
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    N, C = h.shape
    K = indices.shape[1]
    e_local = n_experts // world
    flat = indices.reshape(-1).long()
    order = torch.argsort(flat, stable=True)                       # pairs sorted by global expert
    counts = torch.bincount(flat, minlength=n_experts)             # per expert, this rank's tokens
    recv_counts = torch.empty_like(counts)
    dist.all_to_all_single(recv_counts, counts, group=group)       # [src rank][local expert]
    in_splits = counts.view(world, e_local).sum(1).tolist()        # host sync (baseline only)
    rc = recv_counts.view(world, e_local)
    out_splits = rc.sum(1).tolist()
    send = h[(order // K)]
    recv = _AllToAllRows.apply(send, out_splits, in_splits, group)
    # received rows are ordered (source rank, local expert); tag every row with its local expert
    expert_of_row = torch.repeat_interleave(torch.arange(e_local, device=h.device).repeat(world), rc.reshape(-1))
    ones = torch.ones(recv.shape[0], 1, dtype=scores.dtype, device=h.device)
    y = ops.moe_ffn(recv, w_in, w_out, ones, expert_of_row.view(-1, 1).to(torch.int32))
    back = _AllToAllRows.apply(y, in_splits, out_splits, group)     # rows return in the send order
    sc = scores.reshape(-1)[order].unsqueeze(-1).to(back.dtype)
    out = torch.zeros(N, C, dtype=torch.float32, device=h.device)
    out.index_add_(0, order // K, (back * sc).float())
    return out.to(h.dtype)


# ------------------------------------------------------------------ peer-memory transport
class PeerDispatcher:
    """Per-process state of the pull-based dispatch/combine (symmetric heap buffers, epochs)."""

    _instances = {}

    @classmethod
    def get(cls, group, device, rows_cap: int, C: int, n_experts: int) -> "PeerDispatcher":
        key = (id(group), rows_cap, C, n_experts)
        if key not in cls._instances:
            cls._instances[key] = cls(group, device, rows_cap, C, n_experts)
        return cls._instances[key]

    def __init__(self, group, device, rows_cap: int, C: int, n_experts: int) -> None:
        from archscale_b200.parallel.symm import SymmetricHeap
        self.group, self.device = group, device
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.rows_cap, self.C, self.E = rows_cap, C, n_experts
        self.e_local = n_experts // self.world
        # Rows one rank may have to process.  Routing is not balanced (least of all at initialisation), so
        # the default covers the worst case (every token of every rank lands here); lower it with
        # ARCHSCALE_B200_EP_CAPACITY=<factor over the balanced load> to save memory — an overflow is
        # detected before anything is copied and raises.
        import os
        factor = float(os.environ.get("ARCHSCALE_B200_EP_CAPACITY", self.world))
        self.recv_cap = ((int(rows_cap * min(factor, self.world)) + self.e_local * 256 + 255) // 256) * 256   # + segment padding
        row_bytes = C * 2
        need = 2 * rows_cap * row_bytes + self.recv_cap * row_bytes + 16 * (n_experts + 1) * 4 + (1 << 20)
        self.heap = SymmetricHeap(group, need, device)
        self.ext = self.heap.ext
        a = self.heap.alloc
        self.off_send = [a(rows_cap * row_bytes) for _ in range(2)]        # [0] activations out, [1] results back
        self.off_result = a(self.recv_cap * row_bytes)                      # expert outputs, pulled back by the sources
        self.off_counts = a(n_experts * 4)
        self.off_offsets = a((n_experts + 1) * 4)
        self.off_table = a(self.world * self.e_local * 4)                    # where (src, local expert) starts in my recv
        self.send = [self.heap.tensor(o, (rows_cap, C), torch.bfloat16) for o in self.off_send]
        self.result = self.heap.tensor(self.off_result, (self.recv_cap, C), torch.bfloat16)
        self.counts = self.heap.tensor(self.off_counts, (n_experts,), torch.int32)
        self.offsets = self.heap.tensor(self.off_offsets, (n_experts + 1,), torch.int32)
        self.table = self.heap.tensor(self.off_table, (self.world, self.e_local), torch.int32)
        self.chan = 0
        self.stats = {}                                  # call site → rows received there on earlier steps
        self.margin = float(os.environ.get("ARCHSCALE_B200_EP_MARGIN", "1.25"))
        self.sizing = os.environ.get("ARCHSCALE_B200_EP_SIZING", "exact")       # "exact" | "history" (see receive())
        self.sync_calls = int(os.environ.get("ARCHSCALE_B200_EP_SYNC_CALLS", "8"))

    def exchange(self) -> None:
        self.heap.barrier(self.chan)

    def _rows_to_allocate(self, key) -> Optional[int]:
        """Rows to allocate for what this rank is about to receive at call site ``key``, from the counts seen there on
        earlier steps (read back asynchronously, never waited for); None while there is no estimate yet."""
        st = self.stats[key]
        if st["event"] is not None and st["event"].query():
            st["seen"] = max(int(st["pinned"].item()), int(st["seen"] * 0.98))      # slow decay after a spike
            st["event"] = None
        if st["seen"] <= 0:
            return None
        want = int(st["seen"] * self.margin) + 2 * 256
        return min(((want + 255) // 256) * 256, self.recv_cap)

    def receive(self, e_local: int, key=None) -> tuple:
        """Plan + pull: returns (rows received, in local memory; recv_offsets).  ``key = (site, "fwd" | "bwd")`` names the
        MoE layer and the pass.

        How many rows arrive is known on the device only (the plan kernel sums the peers' counts), and the buffer that
        holds them is kept for the backward pass, so it should not be worst-case sized.  Sizing rules:

        * forward, default: the host reads the total once (4 bytes, one wait per MoE layer and step) and allocates exactly;
        * backward: the gradient rows of a layer are as many as its forward rows were, so the forward's size is reused —
          no read, no wait;
        * forward with ``ARCHSCALE_B200_EP_SIZING=history``: after a site's first calls the size comes from the counts it
          saw on earlier steps times ``ARCHSCALE_B200_EP_MARGIN`` (read back asynchronously, never waited for).  Routing
          that shifts by more than the margin between two steps overflows the buffer: the plan kernel then raises the
          device status word (``STATUS_EP_OVERFLOW``), the pull copies nothing past the buffer and the grouped GEMMs never
          store past it, so the step computes garbage but touches no foreign memory, and the trainer stops at its next
          status check.  Early in training (routing collapses and recovers within a few steps) this mode is not safe."""
        st = self.stats.setdefault(key, {"seen": 0, "event": None, "calls": 0, "last_cap": 0,
                                         "pinned": torch.zeros(1, dtype=torch.int32).pin_memory()})
        st["calls"] += 1
        cap = None
        site, direction = key if isinstance(key, tuple) and len(key) == 2 else (key, "fwd")
        fwd = self.stats.get((site, "fwd")) if direction == "bwd" else None
        if fwd is not None and fwd["last_cap"] > 0:
            cap = fwd["last_cap"]
        elif self.sizing == "history" and st["calls"] > self.sync_calls:
            cap = self._rows_to_allocate(key)
        recv_off = self.ext.ep_plan(self.heap.bases, self.off_counts, self.off_table, self.rank, e_local,
                                    self.recv_cap if cap is None else cap)
        if cap is None:
            used = int(recv_off[-1].item())
            if used > self.recv_cap:
                raise RuntimeError(f"expert-parallel receive overflow: {used} rows > capacity {self.recv_cap}; "
                                   "raise ARCHSCALE_B200_EP_CAPACITY")
            st["seen"] = max(st["seen"], used, 1)
            # rounded up to 8192 rows: sizes that differ a little from step to step then map to the same cached block of
            # the allocator instead of forcing a new cudaMalloc (a device synchronisation) now and then
            cap = min(max(((used + 8191) // 8192) * 8192, 256), max(self.recv_cap, ((used + 255) // 256) * 256))
        elif self.sizing == "history" and st["event"] is None:
            st["pinned"].copy_(recv_off[-1:], non_blocking=True)       # read by a later call, never waited for
            st["event"] = torch.cuda.Event()
            st["event"].record()
        st["last_cap"] = cap
        rows = torch.empty(cap, self.C, dtype=torch.bfloat16, device=self.device)
        self.ext.ep_pull(self.heap.bases, self.off_counts, self.off_offsets, self.off_table, self.off_send[0], rows,
                         self.rank, e_local, recv_off)
        return rows, recv_off


class _EPPeerFn(torch.autograd.Function):
    """Expert-parallel routed FFN with peer-memory dispatch / combine (no NCCL; one 4-byte host read per layer in the
    forward pass to size the receive buffer, none in the backward pass — see :meth:`PeerDispatcher.receive`)."""

    @staticmethod
    def forward(ctx, h, w_in, w_out, scores, indices, n_experts, group, site=None):
        ext = backend.require_extension()
        N, C = h.shape
        K = indices.shape[1]
        E_l, I2, _ = w_in.shape
        I = w_out.shape[2]
        h = h.contiguous()
        sc = scores.float().contiguous()
        counts, offsets, slot_pair, pair_slot = ext.routing_layout(indices.reshape(-1).to(torch.int32).contiguous(), n_experts)
        d = PeerDispatcher.get(group, h.device, slot_pair.numel(), C, n_experts)
        d.counts.copy_(counts)
        d.offsets.copy_(offsets)
        ext.gather_rows(h, slot_pair, None, K, offsets, d.send[0])
        d.exchange()                                                       # every rank's rows and counts are published
        xr, recv_off = d.receive(E_l, key=(site, "fwd"))
        ctx.site = site
        if xr.shape[0] % 256 == 0 and fused_swiglu_enabled():
            h1, a = ext.grouped_gemm_swiglu(xr, w_in.reshape(E_l * I2, C), recv_off, I, True)   # SwiGLU in the epilogue
        else:
            h1 = ext.grouped_gemm_bf16(0, xr, w_in.reshape(E_l * I2, C), recv_off, 0, I2, C)
            a = ext.swiglu_packed_fwd(h1)
        ext.grouped_gemm_bf16(0, a, w_out.reshape(E_l * C, I), recv_off, 0, C, I, None, d.result)
        d.exchange()                                                       # expert outputs are ready everywhere
        yb = torch.empty(slot_pair.numel(), C, dtype=h.dtype, device=h.device)
        ext.ep_return(d.heap.bases, d.off_counts, d.off_offsets, d.off_table, d.off_result, yb, d.rank, E_l, C)
        out = ext.combine_rows(yb, pair_slot, sc, N, K)
        backend.count_launch(14)
        ctx.save_for_backward(xr, h1, a, yb, w_in, w_out, sc, counts, offsets, slot_pair, pair_slot)
        ctx.meta = (N, C, K, E_l, I2, I, n_experts, group, scores.dtype)
        ctx.w_refs = (w_in, w_out)
        return out

    @staticmethod
    def backward(ctx, dout):
        ext = backend.require_extension()
        xr, h1, a, yb, w_in, w_out, sc, counts, offsets, slot_pair, pair_slot = ctx.saved_tensors
        N, C, K, E_l, I2, I, n_experts, group, score_dtype = ctx.meta
        dout = dout.contiguous()
        d = PeerDispatcher.get(group, dout.device, slot_pair.numel(), C, n_experts)
        dscores = ext.pair_dots(yb, dout, pair_slot, K).view(N, K).to(score_dtype)
        d.counts.copy_(counts)
        d.offsets.copy_(offsets)
        ext.gather_rows(dout, slot_pair, sc.reshape(-1), K, offsets, d.send[0])      # dy[slot] = score · dout[token]
        d.exchange()
        dyr, recv_off = d.receive(E_l, key=(ctx.site, "bwd"))
        da = ext.grouped_gemm_bf16(1, dyr, w_out.reshape(E_l * C, I), recv_off, 0, I, C)
        mg_out = getattr(ctx.w_refs[1], "main_grad", None)
        dw_out = ext.grouped_gemm_bf16(2, dyr, a, recv_off, C, I, 0, mg_out)
        dh = ext.swiglu_packed_bwd(h1, da)
        ext.grouped_gemm_bf16(1, dh, w_in.reshape(E_l * I2, C), recv_off, 0, C, I2, None, d.result)
        mg_in = getattr(ctx.w_refs[0], "main_grad", None)
        dw_in = ext.grouped_gemm_bf16(2, dh, xr, recv_off, I2, C, 0, mg_in)
        d.exchange()
        dxs = torch.empty(slot_pair.numel(), C, dtype=dout.dtype, device=dout.device)
        ext.ep_return(d.heap.bases, d.off_counts, d.off_offsets, d.off_table, d.off_result, dxs, d.rank, E_l, C)
        dx = ext.combine_rows(dxs, pair_slot, None, N, K)
        backend.count_launch(14)
        return dx, (None if mg_in is not None else dw_in), (None if mg_out is not None else dw_out), dscores, None, None, None, None


def peer_path_supported(h, w_in, w_out) -> bool:
    return (h.is_cuda and h.dtype == torch.bfloat16 and w_in.dtype == torch.bfloat16 and backend.has("ep_pull")
            and h.shape[1] % 64 == 0 and w_in.shape[1] % 64 == 0 and w_out.shape[2] % 64 == 0)


USE_PEER_TRANSPORT = True


def moe_ffn_expert_parallel(h, w_in, w_out, scores, indices, n_experts: int, group, site=None) -> torch.Tensor:
    """Routed expert FFN with experts sharded over ``group``.  h:(N,C); w_in:(E_l,2I,C); w_out:(E_l,C,I).
    ``site``: any hashable that names the calling layer (receive buffers are sized from that layer's own history)."""
    if group is None or dist.get_world_size(group) == 1:
        return ops.moe_ffn(h, w_in, w_out, scores.to(h.dtype), indices)
    if USE_PEER_TRANSPORT and dist.get_world_size(group) <= 8 and peer_path_supported(h, w_in, w_out):
        return _EPPeerFn.apply(h, w_in, w_out, scores, indices, n_experts, group, site)
    return _moe_ffn_all_to_all(h, w_in, w_out, scores, indices, n_experts, group)
