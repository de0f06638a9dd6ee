"""Hidden-state expert predictors for prefetch: layer-pair heads (MoE-SpeQ style) and probe-point heads (PROBE style).

Both predict, from the residual stream at a SOURCE layer, which routed experts a later TARGET layer will pick, early
enough that an expert missing from the HBM cache can be fetched from host memory before the target layer runs.
One building block, ``ProjectedHead``: a fixed random projection of the hidden state (hidden -> F, never trained, shared
by all heads of a predictor) with a nonlinearity, then a trainable logistic head (F -> experts).  The head is trained
online by mini-batch SGD on (hidden state, routed experts) samples kept in a ring buffer; until ``warm_samples`` have
been seen it predicts nothing.  Everything runs on the CPU in numpy and only produces hints
``(layer, expert, confidence)``; nothing here moves an expert or changes what a layer computes.

``MoeSpeq``   one head per (source, target) pair of MoE layers with target = source + 1 .. source + lookahead.
``Probe``     heads at a few probe layers (default 25 / 50 / 75 % of the depth), each predicting ALL later MoE layers.
Reference counterparts: python/orchestrator/moe_speq.py (per-pair predictor, random projection + ReLU, sigmoid head,
ring buffer, interval training) and python/orchestrator/probe.py (probe points, SiLU features, per-target heads).
"""
from __future__ import annotations

from typing import Dict, Iterable, List, Optional, Sequence, Tuple

import numpy as np

Hint = Tuple[int, int, float]          # (target layer, expert, confidence)


class _Ring:
    def __init__(self, cap: int, feat: int, n_experts: int):
        self.x = np.zeros((cap, feat), np.float32)
        self.y = np.zeros((cap, n_experts), np.float32)
        self.n, self.cap = 0, cap

    def add(self, x: np.ndarray, ids: Iterable[int]):
        i = self.n % self.cap
        self.x[i] = x
        self.y[i] = 0.0
        for e in ids:
            if e >= 0:
                self.y[i, e] = 1.0
        self.n += 1

    def sample(self, rng, m: int):
        idx = rng.integers(0, min(self.n, self.cap), m)
        return self.x[idx], self.y[idx]


class ProjectedHead:
    """Trainable logistic head over features that the owner has already projected."""

    def __init__(self, feat: int, n_experts: int, top_k: int, lr: float, buffer: int, seed: int):
        self.W = np.zeros((feat, n_experts), np.float32)
        self.b = np.full(n_experts, np.log(max(top_k, 1) / max(n_experts - top_k, 1)), np.float32)     # prior: k of E routed
        self.ring = _Ring(buffer, feat, n_experts)
        self.lr = lr
        self.rng = np.random.default_rng(seed)
        self.trained_steps = 0

    def scores(self, f: np.ndarray) -> np.ndarray:
        return 1.0 / (1.0 + np.exp(-(f @ self.W + self.b)))

    def train(self, steps: int, batch: int):
        if self.ring.n == 0:
            return
        for _ in range(steps):
            x, y = self.ring.sample(self.rng, batch)
            g = 1.0 / (1.0 + np.exp(-(x @ self.W + self.b))) - y          # d(BCE)/d(logit)
            self.W -= self.lr * (x.T @ g) / batch
            self.b -= self.lr * g.mean(0)
            self.trained_steps += 1


class _HiddenPredictor:
    """Shared machinery: projection, sample recording, interval training, hint extraction."""
    _act = staticmethod(lambda z: np.maximum(z, 0.0))

    def __init__(self, hidden: int, n_experts: int, top_k: int, pairs: Sequence[Tuple[int, int]], feat: int = 256, lr: float = 0.05,
                 buffer: int = 4096, train_interval: int = 64, train_steps: int = 8, batch: int = 64, warm_samples: int = 128,
                 confidence_threshold: float = 0.5, seed: int = 0):
        rng = np.random.default_rng(seed)
        self.P = (rng.standard_normal((hidden, feat)) / np.sqrt(hidden)).astype(np.float32)
        self.E, self.K, self.feat = n_experts, top_k, feat
        self.heads: Dict[Tuple[int, int], ProjectedHead] = {p: ProjectedHead(feat, n_experts, top_k, lr, buffer, seed + 1 + i) for i, p in enumerate(pairs)}
        self.by_source: Dict[int, List[int]] = {}
        for s, t in pairs:
            self.by_source.setdefault(s, []).append(t)
        self.train_interval, self.train_steps, self.batch = train_interval, train_steps, batch
        self.warm, self.thr = warm_samples, confidence_threshold
        self._feat_cache: Dict[int, np.ndarray] = {}
        self._since_train = 0

    def features(self, hidden_state: np.ndarray) -> np.ndarray:
        h = np.asarray(hidden_state, np.float32)
        h = h / (np.sqrt((h * h).mean()) + 1e-6)                               # scale-free: the residual norm grows with depth
        return self._act(h @ self.P)

    def source_layers(self) -> List[int]:
        return sorted(self.by_source)

    def is_warm(self, source: int, target: int) -> bool:
        return self.heads[(source, target)].ring.n >= self.warm and self.heads[(source, target)].trained_steps > 0

    def observe_hidden(self, layer: int, hidden_state: np.ndarray):
        """Called when the step reaches a source layer; keeps the features until the targets' routing is known."""
        if layer in self.by_source:
            self._feat_cache[layer] = self.features(hidden_state)

    def predict(self, source: int, max_per_layer: Optional[int] = None) -> List[Hint]:
        """Hints for all targets of ``source`` from the hidden state last observed there (empty until warm)."""
        f = self._feat_cache.get(source)
        if f is None:
            return []
        out: List[Hint] = []
        m = max_per_layer or 2 * self.K
        for t in self.by_source[source]:
            if not self.is_warm(source, t):
                continue
            s = self.heads[(source, t)].scores(f)
            top = np.argsort(-s)[:m]
            out.extend((t, int(e), float(s[e])) for e in top if s[e] >= self.thr)
        return out

    def observe_routing(self, target: int, expert_ids: Iterable[int]):
        """Called when a target layer has routed: one training sample for every head that predicts this layer."""
        ids = list(expert_ids)
        for (s, t), head in self.heads.items():
            if t == target and s in self._feat_cache:
                head.ring.add(self._feat_cache[s], ids)

    def end_step(self):
        self._feat_cache.clear()
        self._since_train += 1
        if self._since_train >= self.train_interval:
            self._since_train = 0
            for head in self.heads.values():
                if head.ring.n >= self.batch:
                    head.train(self.train_steps, self.batch)

    def recall(self, source: int, target: int, n_eval: int = 256, m: Optional[int] = None) -> float:
        """Fraction of routed experts inside the top-m scores on the most recent samples of a head (calibration aid)."""
        head = self.heads[(source, target)]
        n = min(head.ring.n, head.ring.cap, n_eval)
        if n == 0:
            return 0.0
        x, y = head.ring.x[:n], head.ring.y[:n]
        s = head.scores(x)
        m = m or 2 * self.K
        top = np.argsort(-s, axis=1)[:, :m]
        hit = np.take_along_axis(y, top, 1).sum()
        return float(hit / max(y.sum(), 1.0))


class MoeSpeq(_HiddenPredictor):
    def __init__(self, hidden: int, n_experts: int, top_k: int, moe_layers: Sequence[int], lookahead: int = 2, **kw):
        layers = sorted(moe_layers)
        pairs = [(s, layers[i + d]) for i, s in enumerate(layers) for d in range(1, lookahead + 1) if i + d < len(layers)]
        super().__init__(hidden, n_experts, top_k, pairs, **kw)


class Probe(_HiddenPredictor):
    _act = staticmethod(lambda z: z / (1.0 + np.exp(-z)))      # SiLU

    def __init__(self, hidden: int, n_experts: int, top_k: int, moe_layers: Sequence[int], n_layers: int,
                 probe_points: Sequence[float] = (0.25, 0.5, 0.75), **kw):
        layers = sorted(moe_layers)
        probes = sorted({min(layers, key=lambda l: abs(l - p * n_layers)) for p in probe_points}) if layers else []
        pairs = [(s, t) for s in probes for t in layers if t > s]
        kw.setdefault("confidence_threshold", 0.6)
        super().__init__(hidden, n_experts, top_k, pairs, **kw)
        self.probe_layers = probes
