"""Host-side planning helpers: a priority work queue and a stateless expert-transfer planner.

``WorkQueue``        priority queue of work items keyed by (request, layer, operation): highest priority first, FIFO among equals, only
                     READY items are handed out, O(1) lookup, cancel-by-request without touching the heap (lazy deletion).
``TransferPlanner``  turns ranked prefetch candidates into the transfers worth issuing in the next planning cycle: skips experts that
                     are resident or already in flight, respects the per-GPU in-flight cap and a per-cycle byte budget derived from the
                     host link bandwidth, delays a transfer whose expert is needed far in the future (just in time: start = time until
                     needed - transfer latency), and routes high-priority experts to the stable zone, the rest to the streaming zone.
                     ``plan_evictions`` asks the cache's eviction order for as many victims as a GPU is short of free slots.
                     It plans only; ``csrc/runtime/transfer_engine.cpp`` owns the queues and the copies.
Reference counterparts: python/orchestrator/work_queue.py and python/orchestrator/transfer_scheduler.py.
"""
from __future__ import annotations

import heapq
import itertools
from dataclasses import dataclass
from typing import Callable, Dict, Hashable, Iterable, List, Optional, Sequence, Set, Tuple

PENDING, READY, RUNNING, DONE, CANCELLED = range(5)
Key = Tuple[Hashable, int, str]                      # (request id, layer, operation)


@dataclass
class WorkItem:
    key: Key
    priority: float
    status: int = READY
    payload: object = None
    seq: int = 0


class WorkQueue:
    def __init__(self):
        self._heap: List[Tuple[float, int, Key]] = []
        self._items: Dict[Key, WorkItem] = {}
        self._by_request: Dict[Hashable, Set[Key]] = {}
        self._seq = itertools.count()

    def __len__(self) -> int:
        return len(self._items)

    def insert(self, key: Key, priority: float, status: int = READY, payload=None) -> WorkItem:
        if key in self._items:
            raise KeyError(f"duplicate work item {key}")
        it = WorkItem(key, priority, status, payload, next(self._seq))
        self._items[key] = it
        self._by_request.setdefault(key[0], set()).add(key)
        heapq.heappush(self._heap, (-priority, it.seq, key))
        return it

    def get(self, key: Key) -> Optional[WorkItem]:
        return self._items.get(key)

    def update_priority(self, key: Key, priority: float):
        it = self._items[key]
        it.priority, it.seq = priority, next(self._seq)
        heapq.heappush(self._heap, (-priority, it.seq, key))          # the stale heap entry is skipped on pop

    def update_status(self, key: Key, status: int):
        it = self._items[key]
        it.status = status
        if status in (DONE, CANCELLED):
            self._drop(key)
        elif status == READY:
            heapq.heappush(self._heap, (-it.priority, it.seq, key))

    def pop(self) -> Optional[WorkItem]:
        """Highest-priority READY item, marked RUNNING; None when nothing is ready."""
        parked = []
        out = None
        while self._heap:
            negp, seq, key = heapq.heappop(self._heap)
            it = self._items.get(key)
            if it is None or it.seq != seq or -negp != it.priority:
                continue                                               # cancelled, finished or re-prioritised since
            if it.status != READY:
                if it.status == PENDING:
                    parked.append((negp, seq, key))
                continue
            it.status, out = RUNNING, it
            break
        for e in parked:
            heapq.heappush(self._heap, e)
        return out

    def pop_n(self, n: int) -> List[WorkItem]:
        out = []
        while len(out) < n:
            it = self.pop()
            if it is None:
                break
            out.append(it)
        return out

    def cancel_by_request(self, request) -> int:
        keys = list(self._by_request.get(request, ()))
        for k in keys:
            self._items[k].status = CANCELLED
            self._drop(k)
        return len(keys)

    def by_status(self, status: int) -> List[WorkItem]:
        return [it for it in self._items.values() if it.status == status]

    def _drop(self, key: Key):
        self._items.pop(key, None)
        s = self._by_request.get(key[0])
        if s is not None:
            s.discard(key)
            if not s:
                del self._by_request[key[0]]


# ------------------------------------------------------------------------------------------------------------------ transfers
ZONE_STABLE, ZONE_STREAMING = 0, 1


@dataclass
class Candidate:
    layer: int
    expert: int
    gpu: int
    priority: float
    needed_in_us: float = 0.0


@dataclass
class PlannedTransfer:
    layer: int
    expert: int
    gpu: int
    zone: int
    priority: float
    start_delay_us: float
    nbytes: int


class TransferPlanner:
    def __init__(self, n_gpus: int, expert_bytes: int, link_gbs: Sequence[float] = (), cycle_budget_us: float = 1000.0, max_inflight_per_gpu: int = 4,
                 min_priority: float = 0.01, stable_zone_threshold: float = 0.7, default_link_gbs: float = 55.0):
        if n_gpus <= 0 or expert_bytes <= 0:
            raise ValueError("n_gpus and expert_bytes must be positive")
        self.G, self.nbytes = n_gpus, expert_bytes
        self.max_inflight, self.min_priority, self.stable_thr = max_inflight_per_gpu, min_priority, stable_zone_threshold
        bw = [link_gbs[g] if g < len(link_gbs) else default_link_gbs for g in range(n_gpus)]
        self.budget = [int(b * 1e3 * cycle_budget_us) for b in bw]    # bytes per planning cycle: GB/s x us = 1e3 bytes

    def plan_transfers(self, candidates: Iterable[Candidate], resident: Dict[int, Set[Tuple[int, int]]], in_flight: Dict[int, Set[Tuple[int, int]]],
                       transfer_latency_us: Optional[Dict[int, float]] = None) -> List[PlannedTransfer]:
        lat = transfer_latency_us or {}
        budget = list(self.budget)
        flying = {g: len(in_flight.get(g, ())) for g in range(self.G)}
        out: List[PlannedTransfer] = []
        seen: Set[Tuple[int, int, int]] = set()
        for c in sorted(candidates, key=lambda c: -c.priority):
            k = (c.layer, c.expert)
            if not 0 <= c.gpu < self.G or c.priority < self.min_priority or (c.gpu, *k) in seen:
                continue
            if k in resident.get(c.gpu, ()) or k in in_flight.get(c.gpu, ()):
                continue
            if flying[c.gpu] >= self.max_inflight or budget[c.gpu] < self.nbytes:
                continue
            delay = max(0.0, c.needed_in_us - lat.get(c.gpu, 0.0))
            out.append(PlannedTransfer(c.layer, c.expert, c.gpu, ZONE_STABLE if c.priority >= self.stable_thr else ZONE_STREAMING, c.priority, delay, self.nbytes))
            budget[c.gpu] -= self.nbytes
            flying[c.gpu] += 1
            seen.add((c.gpu, *k))
        return out

    def plan_evictions(self, required_slots: Dict[int, int], free_slots: Dict[int, int], victims_of: Callable[[int, int], List[Tuple[int, int]]]) -> Dict[int, List[Tuple[int, int]]]:
        """``victims_of(gpu, n)`` returns up to n (layer, expert) victims in the cache's eviction order."""
        out: Dict[int, List[Tuple[int, int]]] = {}
        for g, need in required_slots.items():
            deficit = need - free_slots.get(g, 0)
            if 0 <= g < self.G and deficit > 0:
                out[g] = victims_of(g, deficit)[:deficit]
        return out
