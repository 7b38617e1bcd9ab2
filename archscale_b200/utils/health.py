"""Host-side failure detection between training ranks: heartbeats and an abort flag in a key-value store.

A GPU collective that waits for a rank that has died would only end at the process-group timeout (or never, for a
peer-memory kernel, were its waits not bounded).  So ranks learn about failures on the host, between steps, before
they launch anything that needs the peer:

* every rank ``beat(step)``s once per step;
* a rank that catches an exception publishes ``abort`` (``guard()`` does it) before it exits;
* ``check()`` — called before the next launch — raises :class:`PeerFailure` if an abort was published or a peer's
  heartbeat is older than ``stale_after_s``.

The store is any ``torch.distributed`` store (``TCPStore`` in training, ``FileStore`` / ``HashStore`` in tests).
In-kernel waits are the second line of defence: they are bounded and report through the device status word
(``ops.backend.require_extension().device_status()``), which ``check_device()`` turns into the same exception.
"""
from __future__ import annotations

import contextlib
import time
from typing import Optional


class PeerFailure(RuntimeError):
    """Another rank failed (or stopped sending heartbeats); this rank must stop launching collectives."""


class Heartbeat:
    def __init__(self, store, rank: int, world: int, prefix: str = "health", stale_after_s: float = 120.0) -> None:
        self.store, self.rank, self.world, self.prefix, self.stale_after_s = store, rank, world, prefix, stale_after_s
        self.beat(-1)

    def _key(self, name) -> str:
        return f"{self.prefix}/{name}"

    def beat(self, step: int) -> None:
        self.store.set(self._key(self.rank), f"{step}:{time.time():.3f}")

    def report_failure(self, reason: str) -> None:
        self.store.set(self._key("abort"), f"{self.rank}:{reason[:500]}")

    def aborted(self) -> Optional[str]:
        if self.store.check([self._key("abort")]):
            return self.store.get(self._key("abort")).decode()
        return None

    def check(self) -> None:
        msg = self.aborted()
        if msg is not None:
            raise PeerFailure(f"rank {msg.split(':', 1)[0]} reported a failure: {msg.split(':', 1)[1]}")
        now = time.time()
        for r in range(self.world):
            if r == self.rank or not self.store.check([self._key(r)]):
                continue
            step, stamp = self.store.get(self._key(r)).decode().split(":")
            if now - float(stamp) > self.stale_after_s:
                raise PeerFailure(f"rank {r} sent its last heartbeat {now - float(stamp):.0f} s ago (step {step})")

    @contextlib.contextmanager
    def guard(self):
        """Publish an abort for any exception that leaves the block (including KeyboardInterrupt / SystemExit)."""
        try:
            yield self
        except PeerFailure:
            raise
        except BaseException as e:  # noqa: BLE001
            try:
                self.report_failure(repr(e))
            finally:
                raise


def check_device(ext=None) -> None:
    """Raise :class:`PeerFailure` if a bounded in-kernel wait gave up since the last reset of the status word."""
    if ext is None:
        from archscale_b200.ops import backend
        ext = backend.require_extension()
    code = int(ext.device_status())
    if code != 0:
        names = {1: "shared-memory stage never filled", 2: "shared-memory stage never released", 3: "accumulator never filled",
                 4: "accumulator never released", 5: "a peer never signalled", 6: "bad kernel argument",
                 7: "expert-parallel receive buffer too small for the rows routed to this rank",
                 8: "an index tensor pointed outside its table (the access was skipped)"}
        ext.reset_device_status()
        raise PeerFailure(f"a device-side wait timed out: code {code} ({names.get(code, 'unknown')})")
