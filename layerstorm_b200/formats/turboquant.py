"""TurboQuant 4-bit latent KV: codebook, per-layer rotation and a PyTorch reference quantiser.

A latent row c (d values) is stored as  scale = |c| / sqrt(d)  and 4-bit codes of  Pi (c / |c|) * sqrt(d):
after the random rotation the coordinates are close to N(0, 1), so one fixed 16-level Lloyd-Max quantiser of the
standard normal serves every row.  Pi is a fixed orthogonal matrix per layer (QR of a seeded Gaussian, seed
42 + 7 * layer), folded into W_UK / W_UV at load time so attention runs in the rotated space at no extra cost.
Reference: TurboQuant rows of 386 bytes, codebook config/tq_codebooks/codebook_d512_b4.json, rotation seeds
src/compute/tq_init.h (the levels here are re-derived by Lloyd's iteration, not read from that file).
"""
from __future__ import annotations

import math

import torch

_LEVELS = None


def lloyd_max_gaussian(levels: int = 16, iters: int = 200) -> torch.Tensor:
    """Optimal scalar quantiser of N(0, 1): centroid_j = E[x | t_j < x < t_{j+1}], t_j = midpoints (Lloyd iteration)."""
    global _LEVELS
    if _LEVELS is not None and _LEVELS.numel() == levels:
        return _LEVELS.clone()
    c = torch.linspace(-2.5, 2.5, levels, dtype=torch.float64)
    pdf = lambda x: torch.exp(-0.5 * x * x) / math.sqrt(2 * math.pi)
    cdf = lambda x: 0.5 * (1 + torch.erf(x / math.sqrt(2)))
    for _ in range(iters):
        t = torch.cat([torch.tensor([-40.0], dtype=torch.float64), 0.5 * (c[1:] + c[:-1]), torch.tensor([40.0], dtype=torch.float64)])
        mass = cdf(t[1:]) - cdf(t[:-1])
        c = (pdf(t[:-1]) - pdf(t[1:])) / mass.clamp_min(1e-300)
    _LEVELS = c.float()
    return _LEVELS.clone()


def rotation(dim: int, layer: int) -> torch.Tensor:
    """Orthogonal [dim, dim] fp32 matrix of layer ``layer`` (deterministic across ranks and runs)."""
    g = torch.Generator().manual_seed(42 + 7 * layer)
    q, r = torch.linalg.qr(torch.randn(dim, dim, generator=g, dtype=torch.float64))
    q = q * torch.sign(torch.diagonal(r)).unsqueeze(0)          # fix the sign ambiguity of QR
    return q.float()


def quantise(c: torch.Tensor, rot: torch.Tensor, levels: torch.Tensor):
    """c [n, d] -> (codes uint8 [n, d], scale [n]).  Reference implementation of the append kernel."""
    d = c.shape[-1]
    norm = c.float().norm(dim=-1).clamp_min(1e-15)
    u = (c.float() / norm.unsqueeze(-1)) @ rot.T * math.sqrt(d)
    mids = 0.5 * (levels[1:] + levels[:-1])
    codes = (u.unsqueeze(-1) > mids).sum(-1).to(torch.uint8)
    return codes, norm / math.sqrt(d)


def dequantise(codes: torch.Tensor, scale: torch.Tensor, rot: torch.Tensor, levels: torch.Tensor) -> torch.Tensor:
    """Back to the un-rotated latent (what attention effectively sees)."""
    return (levels[codes.long()] * scale.unsqueeze(-1)) @ rot
