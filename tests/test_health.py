"""Failure detection without a GPU fault: host-side heartbeats / abort flag (gloo ranks), and — on a GPU — a bounded
in-kernel wait that runs out on a flag nothing sets and reports through the status word."""
import os
import tempfile
import time

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from archscale_b200.utils.health import Heartbeat, PeerFailure, check_device



def _free_port() -> int:
    import socket
    with socket.socket() as sk:
        sk.bind(("127.0.0.1", 0))
        return sk.getsockname()[1]

def test_stale_heartbeat_and_abort_flag_are_detected():
    store = dist.HashStore()
    a = Heartbeat(store, 0, 2, stale_after_s=0.2)
    b = Heartbeat(store, 1, 2, stale_after_s=0.2)
    a.check()
    time.sleep(0.3)
    a.beat(1)
    with pytest.raises(PeerFailure, match="rank 1"):
        a.check()
    b.beat(1)
    a.check()
    with pytest.raises(ValueError):
        with b.guard():
            raise ValueError("boom")
    with pytest.raises(PeerFailure, match="boom"):
        a.check()


def _worker(rank, world, port, path, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    hb = Heartbeat(dist.FileStore(path, world), rank, world, stale_after_s=30.0)
    outcome = "finished"
    try:
        with hb.guard():
            for step in range(6):
                if rank == 0 and step == 3:
                    time.sleep(1.0)              # host work of this rank; the peer fails meanwhile
                hb.check()                       # before anything that needs the peers
                if rank == 1 and step == 3:
                    raise RuntimeError("rank 1 lost its data loader")     # fails between steps, nothing in flight
                t = torch.ones(4) * step
                dist.all_reduce(t)
                hb.beat(step)
    except PeerFailure as e:
        outcome = f"peer-failure: {e}"
    except RuntimeError as e:
        outcome = f"raised: {e}"
    q.put((rank, outcome))
    # no destroy_process_group(): the peer is gone, a collective shutdown could block


def test_rank_failure_between_steps_stops_the_other_rank_on_the_host():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    with tempfile.TemporaryDirectory() as d:
        procs = [ctx.Process(target=_worker, args=(r, 2, port, os.path.join(d, "store"), q)) for r in range(2)]
        for p in procs:
            p.start()
        got = dict(q.get(timeout=120) for _ in range(2))
        for p in procs:
            p.join(timeout=60)
    assert got[1].startswith("raised: rank 1 lost")
    assert got[0].startswith("peer-failure: rank 1 reported a failure") and "data loader" in got[0]


@pytest.mark.gpu
def test_bounded_device_wait_times_out_and_context_survives():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    from archscale_b200.ops import backend
    ext = backend.require_extension()
    ext.reset_device_status()
    base = ext.symm_alloc(1 << 16)
    try:
        ext.set_peer_wait_limit_cycles(400_000_000)          # ≈ 0.2 s
        t0 = time.time()
        # a two-"rank" table that maps both ranks to this block: nothing ever posts epoch 1 on channel 5
        ext.symm_wait([base, base], 0, 5, 0, 1)
        torch.cuda.synchronize()
        assert time.time() - t0 < 10.0
        assert ext.device_status() == 5                      # "a peer never signalled"
        with pytest.raises(PeerFailure, match="peer never signalled"):
            check_device(ext)
        assert ext.device_status() == 0
        a = torch.randn(256, 256, device="cuda").bfloat16()
        c = ext.gemm_bf16(a, a, 0, torch.bfloat16, None)      # the context is still usable
        torch.cuda.synchronize()
        assert torch.isfinite(c.float()).all() and ext.device_status() == 0
    finally:
        ext.set_peer_wait_limit_cycles(120_000_000_000)
        ext.symm_free(base)
