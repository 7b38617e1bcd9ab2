"""Out-of-bounds writes, index range checks and run-to-run repeatability of kernels (no memory checker runs on the target GPUs)."""
import pytest
import torch

from archscale_b200 import ops
from archscale_b200.ops import backend, mxfp8, nvfp4
from archscale_b200.utils import canary

pytestmark = pytest.mark.gpu


def test_kernels_with_caller_provided_outputs_stay_inside_them():
    ext = backend.require_extension()
    torch.manual_seed(0)
    # block-scaled GEMMs accumulating into an fp32 matrix whose sizes are not multiples of the 128 x 192 tile
    M, N, K = 300, 520, 512
    a = torch.randn(M, K, device="cuda").bfloat16()
    b = torch.randn(N, K, device="cuda").bfloat16()
    acc, raw = canary.guarded((M, N), torch.float32, "cuda")
    nvfp4.gemm(nvfp4.quantize(a), nvfp4.quantize(b), acc=acc)
    qa, qb = mxfp8.quantize(a), mxfp8.quantize(b)
    mxfp8.gemm(qa[0], qa[1], qb[0], qb[1], acc=acc)
    torch.cuda.synchronize()
    assert canary.guards_intact(acc, raw) and torch.isfinite(acc).all()
    # gathered expert rows written into a caller's buffer (the expert-parallel send buffer is used this way)
    Ntok, C, E, Kt = 333, 256, 7, 3
    x = torch.randn(Ntok, C, device="cuda").bfloat16()
    idx = torch.stack([torch.randperm(E, device="cuda")[:Kt] for _ in range(Ntok)]).to(torch.int32)
    counts, offsets, slot_pair, pair_slot = ext.routing_layout(idx.reshape(-1).contiguous(), E)
    out, raw2 = canary.guarded((slot_pair.numel(), C), torch.bfloat16, "cuda")
    ext.gather_rows(x, slot_pair, None, Kt, offsets, out)
    torch.cuda.synchronize()
    assert canary.guards_intact(out, raw2)
    # cross-entropy in place on a logits chunk with a vocabulary that is not a multiple of the vector width times the block
    logits, raw3 = canary.guarded((257, 1000), torch.bfloat16, "cuda")
    logits.copy_(torch.randn(257, 1000, device="cuda"))
    tgt = torch.randint(0, 1000, (257,), device="cuda")
    ext.cross_entropy_fwd_bwd_(logits, tgt, -100, 0.0, 0.0)
    torch.cuda.synchronize()
    assert canary.guards_intact(logits, raw3)
    assert ext.device_status() == 0


def test_an_index_outside_its_table_is_reported_and_skipped():
    """A corrupted routing table: the kernels record STATUS_INDEX_RANGE and leave the row out.  The bad values still point into
    memory this test owns (spare rows behind the tables' logical ends), so nothing outside the test's tensors is touched even
    where a check were missing."""
    ext = backend.require_extension()
    torch.manual_seed(1)
    Ntok, C, E, Kt, spare = 64, 128, 4, 2, 64
    x_all = torch.randn(Ntok + spare, C, device="cuda").bfloat16()
    x = x_all[:Ntok]                                          # the spare rows sit right behind the logical tensor
    idx = torch.stack([torch.randperm(E, device="cuda")[:Kt] for _ in range(Ntok)]).to(torch.int32)
    counts, offsets, slot_pair, pair_slot = ext.routing_layout(idx.reshape(-1).contiguous(), E)
    good = ext.gather_rows(x, slot_pair, None, Kt, offsets)
    assert ext.device_status() == 0
    bad = slot_pair.clone()
    victim = int((bad >= 0).nonzero()[0])
    bad[victim] = Ntok * Kt + 5                               # pair index past the table; token row Ntok + 2 exists in x_all
    got = ext.gather_rows(x, bad, None, Kt, offsets)
    torch.cuda.synchronize()
    assert ext.device_status() == 8
    assert float(got[victim].float().abs().max()) == 0.0      # skipped: written as a padding row
    used = int(offsets[-1])                                   # rows behind the last expert's segment are never written
    keep = torch.ones(used, dtype=torch.bool, device="cuda")
    keep[victim] = False
    assert torch.equal(got[:used][keep], good[:used][keep])
    ext.reset_device_status()
    # combine / dots with a slot past the row buffer
    y_all = torch.randn(slot_pair.numel() + spare, C, device="cuda").bfloat16()
    y = y_all[:slot_pair.numel()]
    w = torch.rand(Ntok, Kt, device="cuda")
    ref = ext.combine_rows(y, pair_slot, w, Ntok, Kt)
    bad_ps = pair_slot.clone()
    bad_ps[3] = slot_pair.numel() + 1
    out = ext.combine_rows(y, bad_ps, w, Ntok, Kt)
    torch.cuda.synchronize()
    assert ext.device_status() == 8
    t = 3 // Kt
    rows = torch.ones(Ntok, dtype=torch.bool, device="cuda")
    rows[t] = False
    assert torch.equal(out[rows], ref[rows])
    ext.reset_device_status()
    dots = ext.pair_dots(y, torch.randn(Ntok, C, device="cuda").bfloat16(), bad_ps, Kt)
    torch.cuda.synchronize()
    assert ext.device_status() == 8 and float(dots[3]) == 0.0
    ext.reset_device_status()
    assert ext.device_status() == 0


def test_kernels_without_order_dependent_atomics_repeat_bit_for_bit():
    torch.manual_seed(2)
    a = torch.randn(512, 1024, device="cuda").bfloat16()
    b = torch.randn(768, 1024, device="cuda").bfloat16()
    assert canary.bitwise_repeatable(lambda: ops.linear(a, b))
    x = torch.randn(1000, 2048, device="cuda").bfloat16().requires_grad_()
    w = torch.ones(2048, device="cuda").bfloat16().requires_grad_()
    g = torch.randn(1000, 2048, device="cuda").bfloat16()
    assert canary.bitwise_repeatable(lambda: torch.autograd.grad(ops.rms_norm(x, w, 1e-5), (x, w), g))
    q = torch.randn(2, 512, 8, 128, device="cuda").bfloat16()
    k = torch.randn(2, 512, 2, 128, device="cuda").bfloat16()
    v = torch.randn(2, 512, 2, 128, device="cuda").bfloat16()
    with torch.no_grad():
        assert canary.bitwise_repeatable(lambda: ops.attention(q, k, v))
    assert canary.bitwise_repeatable(lambda: nvfp4.quantize_both(a))
    assert canary.bitwise_repeatable(lambda: mxfp8.quantize_both(a))
