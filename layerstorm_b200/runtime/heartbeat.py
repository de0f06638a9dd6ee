"""Rank liveness for the multi-process server: heartbeats through a key-value store, checked by the leader before it announces a call.

Every rank runs a ``Heartbeat`` thread that writes ``hb/<rank> = <beat counter>`` to a store every ``interval_s``.  The leader's
``RankMonitor`` reads the counters on its own thread; a rank whose counter has not moved for ``timeout_s`` is declared failed, and so is
a rank that says goodbye by writing ``-1`` (clean exits between steps are told from crashes).  ``SpmdLeader`` consults the monitor before
every mirrored call and raises ``RankFailure`` instead of launching a step whose in-kernel NVLink waits could only time out (those waits
are bounded and report through an error word, but a host-side verdict is faster, names the rank and keeps the CUDA context clean).
The store is anything with ``set(key, str)`` / ``get(key) -> bytes | str`` (``torch.distributed.TCPStore`` / ``FileStore`` / ``HashStore``),
so the same code runs over the rendezvous store of a torchrun job and over an in-process store in tests.  Nothing here touches a GPU.
The reference runs all GPUs from one process and has no heartbeat between ranks; this component exists because this framework runs one
process per GPU.
"""
from __future__ import annotations

import threading
import time
from typing import Callable, Dict, List, Optional


class RankFailure(RuntimeError):
    def __init__(self, ranks: List[int], why: str):
        super().__init__(f"rank(s) {ranks} {why}")
        self.ranks = ranks


def _get(store, key: str) -> Optional[str]:
    try:
        v = store.get(key)
    except Exception:            # noqa: BLE001 - stores signal a missing key in different ways
        return None
    return v.decode() if isinstance(v, (bytes, bytearray)) else (None if v is None else str(v))


class Heartbeat:
    def __init__(self, store, rank: int, interval_s: float = 0.5):
        self.store, self.rank, self.interval = store, rank, interval_s
        self.beats = 0
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None

    def beat(self):
        self.beats += 1
        self.store.set(f"hb/{self.rank}", str(self.beats))

    def start(self):
        self.beat()

        def loop():
            while not self._stop.wait(self.interval):
                self.beat()
        self._thread = threading.Thread(target=loop, name=f"heartbeat-{self.rank}", daemon=True)
        self._thread.start()
        return self

    def stop(self, goodbye: bool = True):
        self._stop.set()
        if self._thread:
            self._thread.join(timeout=5)
        if goodbye:
            self.store.set(f"hb/{self.rank}", "-1")              # left on purpose, between steps


class RankMonitor:
    def __init__(self, store, ranks: List[int], timeout_s: float = 5.0, clock: Callable[[], float] = time.monotonic):
        self.store, self.ranks, self.timeout, self.clock = store, list(ranks), timeout_s, clock
        now = clock()
        self._last: Dict[int, tuple] = {r: (None, now) for r in self.ranks}      # rank -> (last counter seen, when it last moved)
        self.failed: Dict[int, str] = {}
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None

    def poll(self) -> Dict[int, str]:
        now = self.clock()
        for r in self.ranks:
            if r in self.failed:
                continue
            v = _get(self.store, f"hb/{r}")
            if v == "-1":
                self.failed[r] = "left"
                continue
            seen, when = self._last[r]
            if v is not None and v != seen:
                self._last[r] = (v, now)
            elif now - when > self.timeout:
                self.failed[r] = f"sent no heartbeat for {now - when:.1f} s"
        return self.failed

    def check(self):
        """Raise if any rank has failed (cheap: reads the monitor's verdict, does not touch the store)."""
        if self.failed:
            ranks = sorted(self.failed)
            raise RankFailure(ranks, "; ".join(f"{r}: {self.failed[r]}" for r in ranks))

    def start(self, interval_s: float = 0.5):
        def loop():
            while not self._stop.wait(interval_s):
                self.poll()
        self._thread = threading.Thread(target=loop, name="rank-monitor", daemon=True)
        self._thread.start()
        return self

    def stop(self):
        self._stop.set()
        if self._thread:
            self._thread.join(timeout=5)
