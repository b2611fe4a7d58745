"""Host-side failure detection: heartbeats through the rendezvous store, and step-level deadlines.

The reference has none (a dead rank leaves the others in an NCCL hang). Every rank runs a ``Heartbeat``
thread that bumps ``hb/<rank>`` in a ``torch.distributed`` store; ``check_peers`` (called between steps,
before the next launch) raises ``RankFailure`` naming the ranks whose counter stopped moving, so the job
can stop and restart from the last split checkpoint instead of hanging. Nothing here touches a GPU.
"""
from __future__ import annotations

import threading
import time
from typing import Dict, List, Optional


class RankFailure(RuntimeError):
    def __init__(self, dead: List[int], detail: str = "") -> None:
        super().__init__(f"ranks {dead} stopped sending heartbeats{': ' + detail if detail else ''}")
        self.dead = dead


class OsloCommTimeout(RuntimeError):
    """A device-side bounded wait gave up; ``code`` is the value kernels left in the error word."""

    def __init__(self, code: int) -> None:
        names = {1: "TMA stage never arrived", 2: "shared-memory stage never freed", 3: "accumulator never filled",
                 4: "accumulator never drained", 5: "peer flag never set", 6: "index out of bounds"}
        super().__init__(f"device wait timed out (code {code}: {names.get(code, 'unknown')})")
        self.code = code


def raise_if_device_error(like) -> None:
    """Read the per-device error word (synchronises) and raise ``OsloCommTimeout`` if a kernel gave up."""
    from ..ops import cuda_ops
    code = cuda_ops.device_error_code(like)
    if code:
        cuda_ops.reset_device_error(like)
        raise OsloCommTimeout(code)


class Heartbeat:
    def __init__(self, store, rank: int, world: int, period_s: float = 5.0, misses: int = 6) -> None:
        self.store, self.rank, self.world = store, rank, world
        self.period_s, self.misses = period_s, misses
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self._seen: Dict[int, tuple] = {}
        self._paused = False

    def _key(self, r: int) -> str:
        return f"oslo_b200/hb/{r}"

    def start(self) -> "Heartbeat":
        self.store.add(self._key(self.rank), 1)
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()
        return self

    def _run(self) -> None:
        while not self._stop.wait(self.period_s):
            if not self._paused:
                try:
                    self.store.add(self._key(self.rank), 1)
                except Exception:
                    return

    def pause(self, paused: bool = True) -> None:
        """Test hook: stop beating without stopping the thread (simulates a wedged rank)."""
        self._paused = paused

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=self.period_s + 1)

    def check_peers(self) -> None:
        """Raise ``RankFailure`` for ranks whose counter has not moved for ``misses`` periods."""
        now = time.monotonic()
        dead = []
        for r in range(self.world):
            if r == self.rank:
                continue
            try:
                val = int(self.store.add(self._key(r), 0))
            except Exception as e:  # the store itself is gone
                raise RankFailure([r], f"store unreachable: {e}") from e
            last = self._seen.get(r)
            if last is None or last[0] != val:
                self._seen[r] = (val, now)
            elif now - last[1] > self.period_s * self.misses:
                dead.append(r)
        if dead:
            raise RankFailure(dead)


class StepDeadline:
    """``with StepDeadline(120): train_step()`` raises ``TimeoutError`` from a timer thread's flag when the
    body overran; the check happens on exit and through ``expired`` so the caller can poll between launches."""

    def __init__(self, seconds: float) -> None:
        self.seconds = seconds
        self.expired = False
        self._timer: Optional[threading.Timer] = None

    def __enter__(self) -> "StepDeadline":
        self._timer = threading.Timer(self.seconds, self._fire)
        self._timer.daemon = True
        self._timer.start()
        return self

    def _fire(self) -> None:
        self.expired = True

    def __exit__(self, exc_type, exc, tb) -> None:
        if self._timer is not None:
            self._timer.cancel()
        if self.expired and exc_type is None:
            raise TimeoutError(f"step exceeded its {self.seconds}s deadline")
