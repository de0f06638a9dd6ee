"""Advisory expert-reuse predictor: online ridge regression over routing history.

For every MoE layer and expert it scores how likely the expert is to be routed at the NEXT position, from features of
the routing seen so far; the scores rank prefetch candidates (``pool``) and eviction victims (``evict_scores``).  It is a
pure signal producer: it never decides which experts a layer computes, issues no transfers and is not consulted by the
expert cache unless a caller asks it to (score-then-update, CPU only, allocation-free after construction).

Features per (layer, expert), all causal:
  0 bias | 1 routed at the previous position | 2 fast EMA of routed | 3 slow EMA of routed | 4 routed at the previous
  position in the layer ``lag`` below (the residual stream changes slowly, neighbouring layers agree) | 5 1 / (1 + positions
  since last routed)
The per-layer weights solve a decayed ridge system (A = sum decay^t x x^T + lambda I, b = sum decay^t x y), re-solved in
closed form every ``refresh`` positions.
Reference counterpart: src/prefetch/expert_ridge.h:1-37 (advisory ExpertRidge: open / eviction / manifest heads over
routing-history features with online decayed sufficient statistics).  This is an independent, smaller model; the
reference's trained bundle is not reproduced.
"""
from __future__ import annotations

from typing import Optional

import numpy as np

N_FEAT = 6


class ExpertRidge:
    def __init__(self, n_layers: int, n_experts: int, top_k: int, lag: int = 1, decay: float = 0.999, lam: float = 1.0, refresh: int = 16,
                 fast: float = 0.5, slow: float = 0.05):
        self.J, self.E, self.K, self.lag = n_layers, n_experts, top_k, lag
        self.decay, self.lam, self.refresh, self.fast, self.slow = decay, lam, refresh, fast, slow
        self.w = np.zeros((n_layers, N_FEAT), np.float64)
        self.w[:, 2] = 1.0                                         # before any data: rank by the fast EMA
        self.A = np.tile(np.eye(N_FEAT) * lam, (n_layers, 1, 1))
        self.b = np.zeros((n_layers, N_FEAT), np.float64)
        self.prev = np.zeros((n_layers, n_experts), np.float32)    # routed at the previous position
        self.ema_f = np.zeros((n_layers, n_experts), np.float32)
        self.ema_s = np.zeros((n_layers, n_experts), np.float32)
        self.since = np.full((n_layers, n_experts), 1e6, np.float32)
        self.feat = np.zeros((n_layers, n_experts, N_FEAT), np.float32)
        self.scores = np.zeros((n_layers, n_experts), np.float32)
        self.positions = 0
        self.hits = np.zeros(n_layers, np.int64)                   # calibration: routed experts that were inside the advised pool
        self.seen = np.zeros(n_layers, np.int64)
        self._pool: Optional[np.ndarray] = None

    # ------------------------------------------------------------------ scoring
    def _features(self):
        f = self.feat
        f[..., 0] = 1.0
        f[..., 1] = self.prev
        f[..., 2] = self.ema_f
        f[..., 3] = self.ema_s
        f[..., 4] = 0.0
        if self.lag < self.J:
            f[self.lag:, :, 4] = self.prev[: self.J - self.lag]
        f[..., 5] = 1.0 / (1.0 + self.since)
        return f

    def score(self) -> np.ndarray:
        """[layers, experts] scores for the next position (higher = more likely to be routed)."""
        f = self._features()
        np.einsum("jef,jf->je", f, self.w.astype(np.float32), out=self.scores)
        return self.scores

    def pool(self, m: int) -> np.ndarray:
        """[layers, m] expert ids to keep / prefetch for the next position, best first."""
        s = self.score()
        idx = np.argpartition(-s, min(m, self.E) - 1, axis=1)[:, :m]
        order = np.argsort(-np.take_along_axis(s, idx, 1), axis=1, kind="stable")
        self._pool = np.take_along_axis(idx, order, 1)
        return self._pool

    def evict_scores(self) -> np.ndarray:
        """[layers, experts]: higher = better eviction victim (least likely to be needed soon)."""
        return -self.score()

    # ------------------------------------------------------------------ update (strictly after scoring)
    def step(self, routed: np.ndarray):
        """``routed``: int [layers, top_k] expert ids actually routed at this position (-1 = none)."""
        y = np.zeros((self.J, self.E), np.float32)
        for j in range(self.J):
            ids = routed[j][routed[j] >= 0]
            y[j, ids] = 1.0
            if self._pool is not None:
                self.hits[j] += int(np.isin(ids, self._pool[j]).sum())
                self.seen[j] += len(ids)
        f = self._features().astype(np.float64)
        self.A *= self.decay
        self.b *= self.decay
        self.A += np.einsum("jef,jeg->jfg", f, f) + (1.0 - self.decay) * self.lam * np.eye(N_FEAT)
        self.b += np.einsum("jef,je->jf", f, y.astype(np.float64))
        self.positions += 1
        if self.refresh and self.positions % self.refresh == 0:      # refresh = 0: frozen weights (a trained bundle)
            self.solve()
        self.prev[:] = y
        self.ema_f += self.fast * (y - self.ema_f)
        self.ema_s += self.slow * (y - self.ema_s)
        self.since = np.where(y > 0, 0.0, self.since + 1.0).astype(np.float32)
        self._pool = None

    def solve(self):
        """Re-solve every layer's weights from the accumulated sufficient statistics."""
        for j in range(self.J):
            self.w[j] = np.linalg.solve(self.A[j], self.b[j])

    def reset_history(self):
        """Forget the routing history (a new sequence starts); weights and sufficient statistics stay."""
        self.prev[:] = 0
        self.ema_f[:] = 0
        self.ema_s[:] = 0
        self.since[:] = 1e6
        self._pool = None

    def save_weights(self, path: str, meta: Optional[dict] = None):
        """Weights + the hyper-parameters the features depend on, as one ``.npz`` (written by ``utils/expert_predictor_train.py``)."""
        import json
        np.savez(path, w=self.w, shape=np.array([self.J, self.E, self.K, self.lag]), ema=np.array([self.fast, self.slow]),
                 meta=np.array(json.dumps(meta or {})))

    def load_weights(self, path: str, freeze: bool = True):
        """Install trained weights; with ``freeze`` they are no longer re-solved online."""
        z = np.load(path, allow_pickle=False)
        J, E, K, lag = (int(x) for x in z["shape"])
        if (J, E) != (self.J, self.E) or lag != self.lag:
            raise ValueError(f"predictor weights are for {J} layers x {E} experts (lag {lag}), this model has {self.J} x {self.E} (lag {self.lag})")
        self.w[:] = z["w"]
        self.fast, self.slow = (float(x) for x in z["ema"])
        if freeze:
            self.refresh = 0

    def coverage(self) -> np.ndarray:
        """Per layer: fraction of routed experts that were inside the last advised pools (calibration of ``pool``)."""
        return self.hits / np.maximum(self.seen, 1)
