"""On-box calibration of the expert placement solver's constants.

Measures, with CUDA events after warm-up:
  * host -> device copy rate and latency per (host bank, GPU) with pinned buffers of one expert slot,
  * the grouped expert-FFN compute curve  t(c) = a * c + b * ceil(c / P)  for c experts of one token each
    (least-squares fit over a sweep of c),
  * the cross-device combine cost (one fused all-reduce of a [1, hidden] row) when more than one GPU takes part.
The result is a JSON document (version 2) that ``LoaderSolver.from_calibration`` turns into solver constants.
Modes: ``loaded`` = read a stored file, ``quick`` = few sizes / repetitions, ``full`` = the whole sweep.
Reference: loader calibration (src/core/gpu_loader/loader_calibration.*, JSON v2, modes loaded/quick/full); the
PCIe link warm-up of the reference is replaced by an untimed first copy.
"""
from __future__ import annotations

import json
import time
from typing import Dict, List, Optional, Sequence, Tuple

CALIBRATION_VERSION = 2


def fit_compute_curve(counts: Sequence[int], times_ns: Sequence[float], batch_p: int) -> Tuple[float, float]:
    """Least squares for t = a*c + b*ceil(c/P), a, b >= 0."""
    import numpy as np
    c = np.asarray(counts, dtype=np.float64)
    A = np.stack([c, np.ceil(c / batch_p)], 1)
    sol, *_ = np.linalg.lstsq(A, np.asarray(times_ns, dtype=np.float64), rcond=None)
    a, b = float(sol[0]), float(sol[1])
    if a < 0 or b < 0:                                  # degenerate sweep: fall back to a single-term fit
        a = max(0.0, float((A[:, 0] @ np.asarray(times_ns)) / (A[:, 0] @ A[:, 0])))
        b = 0.0
    return a, b


def measure_h2d(device, nbytes: int, reps: int = 8) -> Tuple[float, float]:
    """(bytes per microsecond, latency ns) of pinned host -> device copies of ``nbytes``."""
    import torch
    src = torch.empty(nbytes, dtype=torch.uint8).pin_memory()
    small = torch.empty(64, dtype=torch.uint8).pin_memory()
    dst = torch.empty(nbytes, dtype=torch.uint8, device=device)
    dst.copy_(src, non_blocking=True)                   # warm-up (link + allocator)
    torch.cuda.synchronize(device)

    def timed(s, d, n):
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(n):
            d.copy_(s, non_blocking=True)
        t1.record()
        torch.cuda.synchronize(device)
        return t0.elapsed_time(t1) * 1e6 / n            # ns per copy
    lat = timed(small, dst[:64], reps * 4)
    big = timed(src, dst, reps)
    rate = nbytes / max(1e-9, (big - lat)) * 1e3        # bytes / us
    return rate, lat


def measure_compute_curve(model, layer: int, counts: Sequence[int], reps: int = 5) -> List[float]:
    """ns per MoE layer call with ``c`` distinct experts active (one token each), on the model's own kernels."""
    import torch
    from ..models.device_model import Workspace
    cfg = model.cfg
    L = model.layers[layer]
    arena = L["arena"]
    out = []
    owned = [e for e, s in enumerate(arena.slot_of.cpu().tolist()) if s >= 0 and e < cfg.n_routed]
    for c in counts:
        c = min(c, len(owned))
        rows = max(1, (c + cfg.top_k - 1) // cfg.top_k)
        ws = Workspace(model, rows, 1, 64)
        ids = torch.full((rows, ws.S), -1, dtype=torch.int32)
        flat = ids.view(-1)
        for j in range(c):
            flat[(j // cfg.top_k) * ws.S + j % cfg.top_k] = owned[j]
        ws.ids.copy_(ids.to(model.device))
        ws.wts.fill_(1.0 / cfg.top_k)
        for _ in range(2):
            model._moe_prepare(arena, ws, rows); model._moe_experts(arena, ws, rows, None)
        torch.cuda.synchronize(model.device)
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(reps):
            model._moe_prepare(arena, ws, rows); model._moe_experts(arena, ws, rows, None)
        t1.record()
        torch.cuda.synchronize(model.device)
        out.append(t0.elapsed_time(t1) * 1e6 / reps)
    return out


def calibrate(model=None, mode: str = "quick", path: Optional[str] = None, batch_p: int = 64) -> dict:
    """Returns the calibration document; ``mode='loaded'`` only reads ``path``."""
    if mode == "loaded":
        if not path:
            raise ValueError("calibration mode 'loaded' needs a path")
        doc = json.load(open(path))
        if doc.get("version") != CALIBRATION_VERSION:
            raise ValueError(f"calibration file version {doc.get('version')} != {CALIBRATION_VERSION}")
        return doc
    import torch
    assert model is not None and mode in ("quick", "full")
    dev = model.device
    layer = next(i for i, L in enumerate(model.layers) if "arena" in L)
    slot_bytes = int(model.layers[layer]["arena"].ef.stride)
    counts = [1, 2, 4, 8] if mode == "quick" else [1, 2, 3, 4, 6, 8, 12, 16, 24, 32, 48, 64]
    rate, lat = measure_h2d(dev, slot_bytes, reps=4 if mode == "quick" else 16)
    times = measure_compute_curve(model, layer, counts, reps=3 if mode == "quick" else 10)
    a, b = fit_compute_curve(counts[: len(times)], times, batch_p)
    doc = {"version": CALIBRATION_VERSION, "mode": mode, "when": time.strftime("%Y-%m-%dT%H:%M:%SZ", time.gmtime()),
           "gpu": torch.cuda.get_device_name(dev), "slot_bytes": slot_bytes, "batch_p": batch_p,
           "devices": [{"a_ns": a, "b_ns": b}],
           "banks": [{"rate_bytes_per_us": [rate], "latency_ns": [lat], "egress_bytes_per_us": rate}],
           "recon_ns": 0.0, "evict_ns": 0.0, "sweep": {"counts": list(counts[: len(times)]), "ns": times}}
    if path:
        with open(path, "w") as fh:
            json.dump(doc, fh, indent=1)
    return doc


def solver_from_calibration(doc: dict):
    """Build the native placement solver from a calibration document."""
    from . import native as rt
    dv, bk = doc["devices"], doc["banks"]
    return rt.LoaderSolver([int(d["a_ns"]) for d in dv], [int(d["b_ns"]) for d in dv],
                           [[int(r) for r in b["rate_bytes_per_us"]] for b in bk], [[int(l) for l in b["latency_ns"]] for b in bk],
                           [int(b["egress_bytes_per_us"]) for b in bk], batch_p=int(doc.get("batch_p", 64)),
                           recon_ns=int(doc.get("recon_ns", 0)), evict_ns=int(doc.get("evict_ns", 0)))
