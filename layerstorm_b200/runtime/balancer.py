"""Host-side placement helpers for the routed experts: a GPU load balancer and a prefetch fuser.

``GpuLoadBalancer`` watches how much routed work every expert attracts (decayed counts per layer) and proposes expert
moves between GPUs that lower the busiest GPU's load, a bounded number of moves per round and only when the imbalance
exceeds a threshold (moving an expert costs a slot image over NVLink or from host memory).  It proposes, it does not
move: the caller applies a move by re-homing the expert in its expert cache / arena.

``PrefetchFuser`` merges the prefetch suggestions of several advisers (router pre-gating of the next layer, same-index
carry-over, the expert-reuse predictor, a speculative draft's routing) into one de-duplicated priority list under a
byte budget; residency and in-flight experts are skipped.
Reference counterparts: python/orchestrator/gpu_load_balancer.py and placement_optimizer.py (cross-GPU work distribution,
timer-gated re-placement) and python/orchestrator/prefetch_fuser.py (fusion of the PreScope / PROBE / MoE-SpeQ / SP-MoE
signals); the reference's production path keeps them advisory as well.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Iterable, List, Optional, Sequence, Set, Tuple

import numpy as np


@dataclass
class Move:
    layer: int
    expert: int
    src: int
    dst: int
    gain: float          # reduction of the busiest GPU's load of that layer


class GpuLoadBalancer:
    def __init__(self, n_layers: int, n_experts: int, n_gpus: int, decay: float = 0.99, threshold: float = 1.15, max_moves: int = 4):
        self.J, self.E, self.G = n_layers, n_experts, n_gpus
        self.decay, self.threshold, self.max_moves = decay, threshold, max_moves
        self.load = np.zeros((n_layers, n_experts), np.float64)
        self.owner = np.tile(np.arange(n_experts) % n_gpus, (n_layers, 1))       # default placement: expert e on GPU e % N

    def observe(self, layer: int, expert_ids: Iterable[int], weight: float = 1.0):
        """One step's routing of a layer (ids < 0 are ignored)."""
        self.load[layer] *= self.decay
        for e in expert_ids:
            if 0 <= e < self.E:
                self.load[layer, e] += weight

    def gpu_loads(self, layer: int) -> np.ndarray:
        return np.bincount(self.owner[layer], weights=self.load[layer], minlength=self.G)

    def imbalance(self, layer: int) -> float:
        g = self.gpu_loads(layer)
        return float(g.max() / max(g.mean(), 1e-12))

    def propose(self, slots_free: Optional[Sequence[int]] = None) -> List[Move]:
        """Moves for the most imbalanced layers, best first.  ``slots_free[g]``: expert slots GPU g can still take (None = unlimited)."""
        free = list(slots_free) if slots_free is not None else None
        owner = self.owner.copy()
        moves: List[Move] = []
        order = sorted(range(self.J), key=lambda j: -self.imbalance(j))
        for j in order:
            while len(moves) < self.max_moves:
                g = np.bincount(owner[j], weights=self.load[j], minlength=self.G)
                if g.mean() <= 0 or g.max() / g.mean() < self.threshold:
                    break
                src, dst = int(g.argmax()), int(g.argmin())
                if free is not None and free[dst] <= 0:
                    break
                gap = g[src] - g[dst]
                cand = [e for e in range(self.E) if owner[j, e] == src and 0 < self.load[j, e] < gap]
                if not cand:
                    break
                e = min(cand, key=lambda x: abs(self.load[j, x] - gap / 2))       # the expert that best halves the gap
                after = g.copy()
                after[src] -= self.load[j, e]
                after[dst] += self.load[j, e]
                new_max = after.max()
                if new_max >= g.max():
                    break
                moves.append(Move(j, e, src, dst, float(g.max() - new_max)))
                owner[j, e] = dst
                if free is not None:
                    free[dst] -= 1
                    free[src] += 1
            if len(moves) >= self.max_moves:
                break
        return moves

    def apply(self, moves: Iterable[Move]):
        for m in moves:
            self.owner[m.layer, m.expert] = m.dst


class PrefetchFuser:
    def __init__(self, slot_bytes: int, budget_bytes: int, source_weight: Optional[Dict[str, float]] = None):
        self.slot_bytes, self.budget = slot_bytes, budget_bytes
        self.weight = {"prescope": 1.0, "same_index": 0.6, "ridge": 0.5, "draft": 0.8}
        if source_weight:
            self.weight.update(source_weight)

    def fuse(self, suggestions: Dict[str, Sequence[Tuple[int, int, float]]], resident: Set[Tuple[int, int]] = frozenset(),
             in_flight: Set[Tuple[int, int]] = frozenset()) -> List[Tuple[int, int, float]]:
        """``suggestions[source]`` = (layer, expert, score in [0, 1]) triples.  Returns (layer, expert, fused score) in issue order:
        fused score = 1 - prod(1 - w_source * score) over the sources that name the expert, nearest layer first on ties, cut at the
        byte budget."""
        miss: Dict[Tuple[int, int], float] = {}
        for src, items in suggestions.items():
            w = self.weight.get(src, 0.5)
            for layer, expert, score in items:
                key = (layer, expert)
                if key in resident or key in in_flight or expert < 0:
                    continue
                p = min(max(w * float(score), 0.0), 1.0)
                miss[key] = miss.get(key, 1.0) * (1.0 - p)
        ranked = sorted(((1.0 - q, -k[0], k) for k, q in miss.items()), reverse=True)
        n = max(0, self.budget // max(self.slot_bytes, 1))
        return [(k[0], k[1], round(s, 6)) for s, _, k in ranked[:n] if s > 0]
