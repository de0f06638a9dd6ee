"""Residual correction for reduced-expert drafts: a small per-layer MLP, trained online, that predicts what the experts a draft pass
leaves out would have added.

A self-speculative draft runs each MoE layer with its top-1 (or top-k') expert only.  During full verification passes both the top-1
output and the full top-k output of a layer are known, so every verified token yields a training sample
    input  = [top-1 output (hidden), gating scores (experts)]        target = full output - top-1 output
and the draft pass then uses  top-1 output + mlp(input)  as the layer's MoE output.  One hidden layer (tanh), trained by mini-batch SGD on
a ring buffer; training writes a shadow copy of the weights that is swapped in whole, so ``predict`` never sees half-updated weights.
Until a layer has ``warm_samples`` samples it predicts a zero correction.
Reference counterpart: python/orchestrator/residual_correction.py (per-layer online MLP, double-buffered weights, ring buffer).
"""
from __future__ import annotations

from typing import Dict, Optional

import numpy as np


class _LayerNet:
    def __init__(self, d_in: int, d_hidden: int, d_out: int, buffer: int, rng):
        self.w = (rng.standard_normal((d_in, d_hidden)).astype(np.float32) / np.sqrt(d_in), np.zeros(d_hidden, np.float32),
                  np.zeros((d_hidden, d_out), np.float32), np.zeros(d_out, np.float32))
        self.x = np.zeros((buffer, d_in), np.float32)
        self.y = np.zeros((buffer, d_out), np.float32)
        self.n = 0
        self.steps = 0

    @staticmethod
    def forward(w, x):
        h = np.tanh(x @ w[0] + w[1])
        return h, h @ w[2] + w[3]


class ResidualCorrection:
    def __init__(self, hidden: int, n_experts: int, mlp_hidden: int = 64, lr: float = 0.05, buffer: int = 2048, batch: int = 64,
                 train_interval: int = 64, train_steps: int = 8, warm_samples: int = 128, seed: int = 0):
        self.H, self.E, self.mh = hidden, n_experts, mlp_hidden
        self.lr, self.buffer, self.batch = lr, buffer, batch
        self.interval, self.train_steps, self.warm = train_interval, train_steps, warm_samples
        self.rng = np.random.default_rng(seed)
        self.layers: Dict[int, _LayerNet] = {}
        self._since = 0

    def _net(self, layer: int) -> _LayerNet:
        if layer not in self.layers:
            self.layers[layer] = _LayerNet(self.H + self.E, self.mh, self.H, self.buffer, self.rng)
        return self.layers[layer]

    def is_warm(self, layer: int) -> bool:
        n = self.layers.get(layer)
        return n is not None and n.n >= self.warm and n.steps > 0

    def predict(self, layer: int, top1_out: np.ndarray, gating: np.ndarray) -> np.ndarray:
        """Correction to add to the reduced-expert output ([hidden] or [rows, hidden]); zeros until the layer is warm."""
        x = np.concatenate([np.asarray(top1_out, np.float32), np.asarray(gating, np.float32)], axis=-1)
        if not self.is_warm(layer):
            return np.zeros(x.shape[:-1] + (self.H,), np.float32)
        return _LayerNet.forward(self.layers[layer].w, x)[1]

    def record(self, layer: int, top1_out: np.ndarray, gating: np.ndarray, full_out: np.ndarray):
        net = self._net(layer)
        i = net.n % self.buffer
        net.x[i, : self.H], net.x[i, self.H:] = top1_out, gating
        net.y[i] = np.asarray(full_out, np.float32) - np.asarray(top1_out, np.float32)
        net.n += 1

    def end_step(self):
        self._since += 1
        if self._since < self.interval:
            return
        self._since = 0
        for net in self.layers.values():
            if net.n >= self.batch:
                self._train(net)

    def _train(self, net: _LayerNet):
        w0, b0, w1, b1 = (a.copy() for a in net.w)                     # shadow copy
        m = min(net.n, self.buffer)
        for _ in range(self.train_steps):
            idx = self.rng.integers(0, m, self.batch)
            x, y = net.x[idx], net.y[idx]
            h = np.tanh(x @ w0 + b0)
            err = (h @ w1 + b1 - y) / self.batch                       # d(0.5 * mse * batch)/d(out)
            gh = (err @ w1.T) * (1.0 - h * h)
            w1 -= self.lr * (h.T @ err)
            b1 -= self.lr * err.sum(0)
            w0 -= self.lr * (x.T @ gh)
            b0 -= self.lr * gh.sum(0)
            net.steps += 1
        net.w = (w0, b0, w1, b1)                                       # swapped in whole

    def error_reduction(self, layer: int, n_eval: int = 256) -> Optional[float]:
        """1 - |target - prediction|^2 / |target|^2 on the most recent samples (0 = no better than no correction)."""
        net = self.layers.get(layer)
        if net is None or net.n == 0:
            return None
        m = min(net.n, self.buffer, n_eval)
        pred = _LayerNet.forward(net.w, net.x[:m])[1]
        den = float((net.y[:m] ** 2).sum())
        return 1.0 - float(((net.y[:m] - pred) ** 2).sum()) / den if den > 0 else 0.0
