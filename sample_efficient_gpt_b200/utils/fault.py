"""Host-side failure handling: step watchdog, non-finite-loss guard, rank heartbeats.

Nothing here touches the device: failures are detected on the host (a step that does not finish,
a loss that is not finite, a peer whose heartbeat stops) and turned into a clean exception or process
exit so that the launcher can restart from the last complete checkpoint
(``training.checkpoint.find_latest``).  The reference has no counterpart (it only zeroes NaN gradients,
training/optimizer.py:66-68).
"""

from __future__ import annotations

import os
import threading
import time

from sample_efficient_gpt_b200.utils.logger import logger


class StepWatchdog:
    """Aborts the process when ``beat()`` is not called for ``timeout_s`` seconds."""

    def __init__(self, timeout_s: float, on_timeout=None, poll_s: float | None = None):
        self.timeout_s = timeout_s
        self.on_timeout = on_timeout or self._abort
        self._last = time.monotonic()
        self._stop = threading.Event()
        self.fired = False
        self._poll = poll_s if poll_s is not None else max(0.05, min(1.0, timeout_s / 4))
        self._thread = threading.Thread(target=self._run, daemon=True)
        if timeout_s > 0:
            self._thread.start()

    def beat(self):
        self._last = time.monotonic()

    def _run(self):
        while not self._stop.wait(self._poll):
            if time.monotonic() - self._last > self.timeout_s:
                self.fired = True
                self.on_timeout()
                return

    @staticmethod
    def _abort():
        logger.error("watchdog: training step did not finish in time; aborting the process")
        os._exit(124)

    def stop(self):
        self._stop.set()


class NonFiniteGuard:
    """Counts consecutive non-finite losses; raises after ``limit`` of them (0 disables)."""

    def __init__(self, limit: int):
        self.limit = limit
        self.streak = 0
        self.total = 0

    def check(self, loss_value: float) -> bool:
        finite = loss_value == loss_value and abs(loss_value) != float("inf")
        if finite:
            self.streak = 0
            return True
        self.streak += 1
        self.total += 1
        if self.limit and self.streak >= self.limit:
            raise FloatingPointError(f"{self.streak} consecutive non-finite losses")
        return False


class RankHeartbeat:
    """Heartbeats through a ``torch.distributed`` key-value store.

    Each rank increments ``hb/<rank>`` from a thread; ``dead_ranks`` lists peers whose counter did not
    move for ``timeout_s``.  Ranks consult it between steps, before launching kernels that wait on peers.
    """

    def __init__(self, store, rank: int, world: int, interval_s: float = 0.5, timeout_s: float = 5.0):
        self.store, self.rank, self.world = store, rank, world
        self.interval_s, self.timeout_s = interval_s, timeout_s
        self._stop = threading.Event()
        self._seen: dict[int, tuple[int, float]] = {}
        self._thread = threading.Thread(target=self._run, daemon=True)
        self.store.add(f"hb/{rank}", 1)
        self._thread.start()

    def _run(self):
        while not self._stop.wait(self.interval_s):
            try:
                self.store.add(f"hb/{self.rank}", 1)
            except Exception:
                return

    def dead_ranks(self) -> list[int]:
        now = time.monotonic()
        dead = []
        for r in range(self.world):
            if r == self.rank:
                continue
            try:
                val = int(self.store.add(f"hb/{r}", 0))
            except Exception:
                dead.append(r)
                continue
            prev = self._seen.get(r)
            if prev is None or prev[0] != val:
                self._seen[r] = (val, now)
            elif now - prev[1] > self.timeout_s:
                dead.append(r)
        return dead

    def stop(self):
        self._stop.set()
