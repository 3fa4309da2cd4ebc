"""Host-side peer health: heartbeats through the rendezvous store.

Every rank bumps ``hb/<rank>`` in the process group's store from a daemon thread; before a step a
rank can call ``check_peers()``, which raises ``PeerFailure`` when some peer's counter has not moved
for ``stale_s`` seconds (the peer raised, exited, or hangs on the host). The training engine uses it
together with the step watchdog: a failed peer is noticed *between* steps, before the next
collective is launched, and the process exits non-zero so the launcher can restart the job from
the newest complete checkpoint. The reference has no failure detection (lset/cli.py:56-67)."""
from __future__ import annotations

import threading
import time
from typing import Dict, Optional


class PeerFailure(RuntimeError):
    pass


class RankHeartbeat:
    def __init__(self, store, rank: int, world: int, interval_s: float = 0.5, stale_s: float = 5.0,
                 prefix: str = "hb"):
        self.store, self.rank, self.world = store, rank, world
        self.interval_s, self.stale_s, self.prefix = interval_s, stale_s, prefix
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self._seen: Dict[int, tuple] = {}

    def _key(self, r: int) -> str:
        return f"{self.prefix}/{r}"

    def start(self) -> None:
        self.store.add(self._key(self.rank), 1)
        self._thread = threading.Thread(target=self._run, name="lset-b200-heartbeat", daemon=True)
        self._thread.start()

    def _run(self) -> None:
        while not self._stop.wait(self.interval_s):
            try:
                self.store.add(self._key(self.rank), 1)
            except Exception:  # the store went away: the job is ending
                return

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2.0)

    def stale_peers(self):
        now = time.monotonic()
        stale = []
        for r in range(self.world):
            if r == self.rank:
                continue
            try:
                count = int(self.store.add(self._key(r), 0))
            except Exception:
                stale.append(r)
                continue
            last = self._seen.get(r)
            if last is None or last[0] != count:
                self._seen[r] = (count, now)
            elif now - last[1] > self.stale_s:
                stale.append(r)
        return stale

    def check_peers(self) -> None:
        stale = self.stale_peers()
        if stale:
            raise PeerFailure(f"rank {self.rank}: no heartbeat from rank(s) {stale} for more than "
                              f"{self.stale_s:.1f} s")
