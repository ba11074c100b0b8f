"""Host-side failure detection: a store-based heartbeat between ranks and a per-step watchdog.

Nothing here touches a GPU. A rank publishes "I finished step s" in the job's key-value store;
before launching the next step every rank checks that all peers got there within a deadline and
raises :class:`RankFailure` (naming the silent ranks) instead of entering a collective that would
never complete. The watchdog is a thread that fires a callback when a step overruns its deadline
(the trainer uses it to write an emergency checkpoint and exit). Device-side waits are bounded on
their own (see ``csrc/kernels/sm100.cuh``); the two mechanisms together mean no rank hangs forever.
"""
from __future__ import annotations

import threading
import time


class RankFailure(RuntimeError):
    def __init__(self, missing, step):
        super().__init__(f"ranks {sorted(missing)} did not reach step {step}")
        self.missing = sorted(missing)
        self.step = step


class Heartbeat:
    def __init__(self, store, rank: int, world: int, prefix: str = "cai/hb"):
        self.store, self.rank, self.world, self.prefix = store, rank, world, prefix

    def beat(self, step: int):
        self.store.set(f"{self.prefix}/{self.rank}", str(step))

    def progress(self, rank: int) -> int:
        try:
            if not self.store.check([f"{self.prefix}/{rank}"]):
                return -1
            return int(self.store.get(f"{self.prefix}/{rank}"))
        except Exception:
            return -1

    def check(self, step: int, timeout: float = 5.0, poll: float = 0.02):
        """Block until every rank has published ``>= step`` or raise RankFailure after ``timeout``.

        Returns ``(waited_s, last_rank)``: how long this rank stood at the check and which peer arrived last (a
        straggler shows up here as a repeated ``last_rank`` with a wait that is a large share of the step time)."""
        t0 = time.monotonic()
        deadline = t0 + timeout
        missing = set(range(self.world))
        last_rank = self.rank
        while True:
            still = {r for r in missing if self.progress(r) < step}
            others = (missing - still) - {self.rank}
            if others:
                last_rank = max(others)     # later batches of arrivals overwrite earlier ones
            missing = still
            if not missing:
                return time.monotonic() - t0, last_rank
            if time.monotonic() > deadline:
                raise RankFailure(missing, step)
            time.sleep(poll)


class Watchdog:
    """Calls ``on_expire()`` once if ``arm()`` is not followed by ``disarm()`` within the deadline."""

    def __init__(self, deadline_s: float, on_expire):
        self.deadline_s, self.on_expire = deadline_s, on_expire
        self._lock = threading.Lock()
        self._armed_at = None
        self._stop = False
        self.fired = False
        self._t = threading.Thread(target=self._run, daemon=True)
        self._t.start()

    def arm(self):
        with self._lock:
            self._armed_at = time.monotonic()

    def disarm(self):
        with self._lock:
            self._armed_at = None

    def close(self):
        self._stop = True
        self._t.join(timeout=1.0)

    def _run(self):
        while not self._stop:
            time.sleep(min(0.01, self.deadline_s / 4))
            with self._lock:
                late = self._armed_at is not None and time.monotonic() - self._armed_at > self.deadline_s
                if late:
                    self._armed_at = None
            if late and not self.fired:
                self.fired = True
                self.on_expire()
