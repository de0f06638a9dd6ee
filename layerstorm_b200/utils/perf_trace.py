"""Stage tracing and the trace report ("x-ray table" + JSON sidecar).

``LS_PERF_TRACE=1`` makes ``serve.py`` wrap its engine in ``TracedEngine``: every engine call leaves a begin and an end
record (32 bytes each, steady-clock ns, stage tag, key = rows or tokens of the call, token = call sequence number) in
the native preallocated trace ring (csrc/runtime/ipc.cpp); at shutdown the ring is dumped as CSV to
``LS_PERF_TRACE_OUT`` (default ``lsb_perf_trace.csv``) and the report is written next to it.

    python -m layerstorm_b200.utils.perf_trace report lsb_perf_trace.csv            # table on stdout, <csv>.json sidecar

Reference counterpart: src/core/perf_trace.h:26-71 (record ring, stage tags, CSV dump at shutdown) and perf_report.*
(x-ray table + JSON sidecar).
"""
from __future__ import annotations

import contextlib
import csv
import json
import os
import sys
from typing import Any, Dict, Iterable, List, Optional

# span name -> (begin tag, end tag)
SPANS = {"prefill": (1, 2), "decode": (3, 4), "forward_rows": (5, 6), "fork_sequence": (7, 8), "rewind": (9, 10), "request": (11, 12),
         "expert_fetch": (13, 14), "free_sequence": (15, 16), "create_sequence": (17, 18), "hibernate": (19, 20), "resume": (21, 22)}
_BEGIN = {b: n for n, (b, _) in SPANS.items()}
_END = {e: n for n, (_, e) in SPANS.items()}


def enabled(env: Optional[dict] = None) -> bool:
    env = os.environ if env is None else env
    return env.get("LS_PERF_TRACE", "") not in ("", "0", "false", "False")


def out_path(env: Optional[dict] = None) -> str:
    env = os.environ if env is None else env
    return env.get("LS_PERF_TRACE_OUT") or "lsb_perf_trace.csv"


class Tracer:
    def __init__(self, capacity: int = 1 << 20, gpu: int = 0):
        from ..runtime import native as rt
        self.ring = rt.PerfTrace(capacity)
        self.gpu = gpu
        self._seq = 0

    @contextlib.contextmanager
    def span(self, name: str, key: int = 0):
        b, e = SPANS[name]
        self._seq += 1
        tok = self._seq
        self.ring.record(b, self.gpu, tok & 0xFFFFFFFF, key, tok)
        try:
            yield
        finally:
            self.ring.record(e, self.gpu, tok & 0xFFFFFFFF, key, tok)

    def dump(self, path: str) -> dict:
        """CSV + report sidecar; returns the report."""
        self.ring.dump_csv(path)
        rep = report(path)
        rep["dropped_records"] = self.ring.dropped()
        with open(os.path.splitext(path)[0] + ".json", "w") as fh:
            json.dump(rep, fh, indent=1)
        return rep


class TracedEngine:
    """Engine facade that brackets the traced calls with begin / end records; everything else passes through."""

    def __init__(self, engine, tracer: Tracer):
        object.__setattr__(self, "_engine", engine)
        object.__setattr__(self, "_tracer", tracer)

    def __getattr__(self, name: str) -> Any:
        attr = getattr(self._engine, name)
        if name in SPANS and callable(attr):
            def traced(*args, **kwargs):
                key = 0
                if name in ("prefill", "forward_rows") and len(args) > 1:
                    key = len(args[1])                         # tokens in the call
                elif name == "decode" and args:
                    key = len(args[0])                         # rows in the step
                with self._tracer.span(name, key):
                    return attr(*args, **kwargs)
            return traced
        return attr

    def __setattr__(self, name: str, value: Any):
        setattr(self._engine, name, value)


def _pct(sorted_vals: List[float], q: float) -> float:
    if not sorted_vals:
        return 0.0
    i = min(len(sorted_vals) - 1, max(0, int(round(q * (len(sorted_vals) - 1)))))
    return sorted_vals[i]


def report(csv_path: str) -> dict:
    """Pair begin / end records by (stage, token) and aggregate per span: calls, total ms, mean / p50 / p99 us, items per second
    (key = tokens or rows of the call)."""
    open_at: Dict[tuple, tuple] = {}
    dur: Dict[str, List[float]] = {}
    keys: Dict[str, int] = {}
    t_min, t_max, n = None, None, 0
    with open(csv_path) as fh:
        for row in csv.DictReader(fh):
            ns, stage, tok, key = int(row["ns"]), int(row["stage"]), int(row["token"]), int(row["key"])
            n += 1
            t_min = ns if t_min is None else min(t_min, ns)
            t_max = ns if t_max is None else max(t_max, ns)
            if stage in _BEGIN:
                open_at[(_BEGIN[stage], tok)] = (ns, key)
            elif stage in _END:
                name = _END[stage]
                b = open_at.pop((name, tok), None)
                if b is not None:
                    dur.setdefault(name, []).append((ns - b[0]) / 1e3)
                    keys[name] = keys.get(name, 0) + b[1]
    spans = {}
    wall_ms = ((t_max - t_min) / 1e6) if n else 0.0
    for name, d in dur.items():
        d.sort()
        tot_ms = sum(d) / 1e3
        spans[name] = {"calls": len(d), "total_ms": round(tot_ms, 3), "share_of_wall": round(tot_ms / wall_ms, 4) if wall_ms else 0.0,
                       "mean_us": round(sum(d) / len(d), 2), "p50_us": round(_pct(d, 0.5), 2), "p99_us": round(_pct(d, 0.99), 2),
                       "items": keys.get(name, 0), "items_per_s": round(keys.get(name, 0) / (tot_ms / 1e3), 1) if tot_ms > 0 else 0.0}
    return {"records": n, "wall_ms": round(wall_ms, 3), "unmatched_begins": len(open_at), "spans": spans}


def format_table(rep: dict) -> str:
    lines = [f"{'span':<16}{'calls':>8}{'total ms':>12}{'% wall':>8}{'mean us':>11}{'p50 us':>11}{'p99 us':>11}{'items/s':>12}"]
    for name, s in sorted(rep["spans"].items(), key=lambda kv: -kv[1]["total_ms"]):
        lines.append(f"{name:<16}{s['calls']:>8}{s['total_ms']:>12.3f}{100 * s['share_of_wall']:>8.1f}{s['mean_us']:>11.1f}{s['p50_us']:>11.1f}"
                     f"{s['p99_us']:>11.1f}{s['items_per_s']:>12.1f}")
    lines.append(f"records {rep['records']}, wall {rep['wall_ms']:.1f} ms, unmatched begins {rep['unmatched_begins']}")
    return "\n".join(lines)


def main(argv: Optional[Iterable[str]] = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if len(argv) < 2 or argv[0] != "report":
        print("usage: python -m layerstorm_b200.utils.perf_trace report <trace.csv> [-o sidecar.json]", file=sys.stderr)
        return 2
    rep = report(argv[1])
    out = argv[argv.index("-o") + 1] if "-o" in argv else os.path.splitext(argv[1])[0] + ".json"
    with open(out, "w") as fh:
        json.dump(rep, fh, indent=1)
    print(format_table(rep))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
