"""Host-side failure detection for multi-rank runs.

Collectives hang when a peer dies. Two mechanisms make a dead or stuck rank visible on the host BEFORE the next
kernel or collective is launched, without any device-side waiting:

* ``Heartbeat``: every rank writes a monotonically increasing counter and a wall-clock stamp under its own key of the
  rendezvous store (``torch.distributed.TCPStore`` or the default store of the process group) from a daemon thread;
  ``missing_peers(max_age)`` lists ranks whose stamp is older than ``max_age`` seconds. A rank that leaves cleanly
  calls ``leave()``, which peers see as an explicit departure rather than a timeout.
* ``guarded_step``: runs one training step and converts a collective timeout / connection error into
  ``PeerFailure`` naming the ranks that stopped beating, after which the caller can checkpoint and exit or shrink the
  group. Faults are never provoked on a GPU: tests inject failures on the host (a rank that raises, exits or stops
  beating).
"""
from __future__ import annotations

import threading
import time
from typing import Callable

from ..base.exceptions import OperationError

__all__ = ["Heartbeat", "PeerFailure", "guarded_step"]


class PeerFailure(OperationError):
    def __init__(self, message: str, ranks: list[int]):
        super().__init__(message)
        self.ranks = ranks


class Heartbeat:
    def __init__(self, store, rank: int, world_size: int, interval: float = 1.0, prefix: str = "opake/hb"):
        self.store, self.rank, self.world, self.interval, self.prefix = store, rank, world_size, interval, prefix
        self._stop = threading.Event()
        self._count = 0
        self._thread: threading.Thread | None = None
        self._beat()

    def _key(self, rank: int) -> str:
        return f"{self.prefix}/{rank}"

    def _beat(self) -> None:
        self._count += 1
        self.store.set(self._key(self.rank), f"{self._count}:{time.time():.3f}")

    def start(self) -> "Heartbeat":
        def loop():
            while not self._stop.wait(self.interval):
                try:
                    self._beat()
                except Exception:        # the store itself is gone: nothing more to report
                    return
        self._thread = threading.Thread(target=loop, name="opake-heartbeat", daemon=True)
        self._thread.start()
        return self

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2 * self.interval + 1)

    def leave(self) -> None:
        """Announces a clean departure (between steps, with nothing in flight)."""
        self.stop()
        self.store.set(self._key(self.rank), "left:0")

    def peer_state(self, rank: int) -> tuple[str, float]:
        """``("alive" | "left" | "unknown", age in seconds)``."""
        try:
            raw = self.store.get(self._key(rank)).decode()
        except Exception:
            return "unknown", float("inf")
        tag, stamp = raw.split(":", 1)
        if tag == "left":
            return "left", 0.0
        return "alive", max(0.0, time.time() - float(stamp))

    def missing_peers(self, max_age: float) -> list[int]:
        out = []
        for r in range(self.world):
            if r == self.rank:
                continue
            state, age = self.peer_state(r)
            if state != "alive" or age > max_age:
                out.append(r)
        return out


def guarded_step(step: Callable[[], object], heartbeat: Heartbeat | None = None, max_age: float = 10.0):
    """Runs ``step()``; before it, refuses to start if a peer is already missing; a failure inside it is re-raised as
    ``PeerFailure`` when the heartbeat shows that a peer is gone (otherwise unchanged)."""
    if heartbeat is not None:
        gone = heartbeat.missing_peers(max_age)
        if gone:
            raise PeerFailure(f"ranks {gone} are not alive; not launching the next step", gone)
    try:
        return step()
    except PeerFailure:
        raise
    except Exception as e:      # noqa: BLE001 - classified by the heartbeat
        if heartbeat is not None:
            time.sleep(min(max_age, 2 * heartbeat.interval))
            gone = heartbeat.missing_peers(max_age)
            if gone:
                raise PeerFailure(f"step failed and ranks {gone} stopped responding: {e}", gone) from e
        raise
