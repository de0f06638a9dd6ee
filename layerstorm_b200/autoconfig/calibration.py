"""Speed capabilities from measurements instead of defaults.

The solver's step-time model uses three bandwidths of ``HardwareInfo`` (HBM copy, NVLink peer copy, pinned host -> device).  Their
defaults are measurements of one B200 pool; ``apply_calibration`` replaces them with what THIS machine measured:
  * the engine's loader calibration document (``runtime/calibration.py``: ``banks[*].rate_bytes_per_us`` is the host -> device rate of
    an expert slot image, ``devices[*].a_ns / b_ns`` the grouped-GEMM cost curve), and / or
  * a peaks document ``{"hbm_gbs": ..., "nvlink_gbs": ..., "h2d_gbs": ...}`` (any subset).
Values outside a plausible range are ignored and reported, so a broken measurement cannot steer the derivation.
Reference counterpart: python/autoconfig/calibration.py (GPU speed capabilities from the engine's own calibration).
"""
from __future__ import annotations

import copy
from typing import List, Tuple

from .hwdetect import HardwareInfo

_RANGE = {"hbm_gbs": (500.0, 16000.0), "nvlink_gbs": (20.0, 2000.0), "h2d_gbs": (2.0, 500.0)}


def apply_calibration(hw: HardwareInfo, doc: dict) -> Tuple[HardwareInfo, List[str]]:
    """Returns (a copy of ``hw`` with measured bandwidths, notes on what was taken or rejected)."""
    out, notes = copy.deepcopy(hw), []
    cand = {k: doc[k] for k in _RANGE if isinstance(doc.get(k), (int, float))}
    banks = doc.get("banks")
    if banks and "h2d_gbs" not in cand:
        rates = [r for b in banks for r in b.get("rate_bytes_per_us", []) if r]
        if rates:
            cand["h2d_gbs"] = min(rates) / 1e3                  # bytes/us = MB/s; the slowest bank bounds a GPU's fetches
    for k, v in cand.items():
        lo, hi = _RANGE[k]
        if lo <= v <= hi:
            notes.append(f"{k}: {getattr(out, k):.0f} -> {v:.0f} GB/s (measured)")
            setattr(out, k, float(v))
        else:
            notes.append(f"{k}: measured {v:.1f} GB/s is outside [{lo:.0f}, {hi:.0f}] and was ignored")
    dv = doc.get("devices")
    if dv:
        notes.append(f"expert GEMM cost curve: a = {dv[0].get('a_ns', 0) / 1e3:.1f} us per call, b = {dv[0].get('b_ns', 0) / 1e3:.2f} us per expert")
    return out, notes
