"""The peer-memory kernels on ONE GPU: both "ranks'" heaps are buffers of the same device, and only kernels that never
wait for another launch are run (the pulls, the piece copies, and the fused all-gather→GEMM kernels, whose waits are on
flags that their own copier CTAs set).  The cross-rank versions of these checks need two GPUs (``tests/test_multigpu.py``);
this file makes the same device code run, against PyTorch oracles, wherever one B200 is present."""
import pytest
import torch

from archscale_b200.ops import backend

pytestmark = pytest.mark.gpu


def _ext():
    return backend.require_extension()


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-20)).item()


def test_allgather_and_reduce_scatter_pull_loopback():
    ext = _ext()
    torch.manual_seed(0)
    S = 256 * 1024 + 64                                   # elements per shard, not a multiple of the kernels' chunk
    shards = [torch.randn(S, device="cuda").bfloat16() for _ in range(2)]
    bases = [t.data_ptr() for t in shards]
    for rank in range(2):
        dst = torch.empty(2 * S, device="cuda", dtype=torch.bfloat16)
        ext.allgather_pull(bases, 0, dst, S * 2, rank, 32)
        assert torch.equal(dst, torch.cat(shards))
    fulls = [torch.randn(2 * S, device="cuda") for _ in range(2)]
    bases = [t.data_ptr() for t in fulls]
    for rank in range(2):
        out = torch.empty(S, device="cuda")
        ext.reduce_scatter_pull(bases, 0, out, rank, 0.5, False, 64)
        ref = 0.5 * (fulls[0][rank * S:(rank + 1) * S] + fulls[1][rank * S:(rank + 1) * S])
        assert torch.allclose(out, ref, atol=1e-6, rtol=1e-6)
        acc = torch.ones(S, device="cuda")
        ext.reduce_scatter_pull(bases, 0, acc, rank, 0.5, True, 64)
        assert torch.allclose(acc, ref + 1, atol=1e-6, rtol=1e-6)
    assert ext.device_status() == 0


def test_pull_pieces_loopback():
    """The owner-only Muon transport: a table of (source rank, source range, destination range) copies."""
    from archscale_b200.parallel.symm import SymmetricContext
    ext = _ext()
    torch.manual_seed(1)
    n = 40_000 * 8
    bufs = [torch.randn(n, device="cuda").bfloat16() for _ in range(2)]
    bases = [t.data_ptr() for t in bufs]
    pieces = [(1, 0, 8, 8 * 5000), (0, 8 * 100, 8 * 6000, 8 * 33000), (1, 8 * 39000, 8 * 39500, 8 * 500)]
    table = SymmetricContext._piece_table(pieces, rank=0, world=2, device=torch.device("cuda"))
    assert table is not None and int((table[:, 2] & 0xffffffff).max()) <= 4096
    dst = torch.zeros(n, device="cuda", dtype=torch.bfloat16)
    ext.pull_pieces(bases, 0, dst, table, 48)
    ref = torch.zeros_like(dst)
    for r, s, d, c in pieces:
        ref[d:d + c] = bufs[r][s:s + c]
    assert torch.equal(dst, ref)


@pytest.mark.parametrize("rank", [0, 1])
def test_fused_allgather_gemm_loopback(rank):
    """FSDP form: the weight's flat shards are pulled by copier CTAs of the same launch that multiplies with them."""
    ext = _ext()
    torch.manual_seed(2)
    M, N, K = 512, 768, 1024
    shard_elems = N * K // 2 + 128 * 1024                 # the gathered buffer holds W (N×K) at element 0 and more behind it
    shards = [(0.05 * torch.randn(shard_elems, device="cuda")).bfloat16() for _ in range(2)]
    bases = [t.data_ptr() for t in shards]
    a = torch.randn(M, K, device="cuda").bfloat16()
    dst = torch.zeros(2 * shard_elems, device="cuda", dtype=torch.bfloat16)
    flags = torch.zeros((dst.numel() * 2 + 256 * 1024 - 1) // (256 * 1024), dtype=torch.int32, device="cuda")
    for epoch in (1, 2):                                   # the second call reuses the flags with the next epoch
        dst.zero_()
        y = ext.ag_gemm(a, bases, 0, dst, shard_elems * 2, 0, N, flags, epoch, rank, 16)
        full = torch.cat(shards)
        assert torch.equal(dst, full)
        ref = a.float() @ full[:N * K].view(N, K).float().t()
        assert _rel(y, ref) < 1e-2
    assert ext.device_status() == 0


@pytest.mark.parametrize("rank", [0, 1])
def test_fused_allgather_a_gemm_loopback(rank):
    """Tensor-parallel form: the activations' row chunks are gathered by the launch that multiplies them with the local weight."""
    ext = _ext()
    torch.manual_seed(3)
    rows_local, K, N = 1024, 512, 640
    chunks = [torch.randn(rows_local, K, device="cuda").bfloat16() for _ in range(2)]
    bases = [t.data_ptr() for t in chunks]
    b = (0.05 * torch.randn(N, K, device="cuda")).bfloat16()
    flags = torch.zeros((2 * rows_local * K * 2 + 256 * 1024 - 1) // (256 * 1024), dtype=torch.int32, device="cuda")
    a_full, y = ext.ag_a_gemm(bases, 0, rows_local, b, flags, 1, rank, 16)
    ref_a = torch.cat(chunks)
    assert torch.equal(a_full, ref_a)
    assert _rel(y, ref_a.float() @ b.float().t()) < 1e-2
    assert ext.device_status() == 0
