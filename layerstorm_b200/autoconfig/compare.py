"""Champion comparison: is a derived configuration at least as good as a hand-tuned one?

Both arms are measured with the same benchmark (``bench.py`` lines, or the ``benchmark`` reports of this package: one JSON object with
``value``, ``higher_is_better`` and optional named sub-metrics under ``extra``), on the same machine.  The candidate passes when every
compared metric is within ``tolerance`` of the champion's (better counts as within); the report lists each metric's ratio so that a
failing derivation names what it lost.  Configurations may be passed too: their differing leaf paths are listed beside the numbers.

    python -m layerstorm_b200.autoconfig.compare champion_bench.json candidate_bench.json [--tolerance 0.03] \
        [--champion-config a.json --candidate-config b.json]

Reference counterpart: python/autoconfig/compare.py (the acceptance instrument of the autoconfig: derived recipe vs champion).
"""
from __future__ import annotations

import argparse
import json
import sys
from typing import Any, Dict, List, Optional, Tuple


def _last_json_line(path: str) -> dict:
    obj = None
    with open(path) as fh:
        txt = fh.read()
    try:
        return json.loads(txt)
    except ValueError:
        pass
    for line in txt.splitlines():
        line = line.strip()
        if line.startswith("{"):
            try:
                obj = json.loads(line)
            except ValueError:
                continue
    if obj is None:
        raise ValueError(f"{path}: no JSON object found")
    return obj


def metrics_of(rep: dict) -> Dict[str, Tuple[float, bool]]:
    """name -> (value, higher_is_better)."""
    out: Dict[str, Tuple[float, bool]] = {}
    hib = bool(rep.get("higher_is_better", True))
    if isinstance(rep.get("value"), (int, float)):
        out[str(rep.get("metric", "value"))] = (float(rep["value"]), hib)
    e2e = rep.get("e2e")
    if isinstance(e2e, dict) and isinstance(e2e.get("value"), (int, float)):
        out["e2e"] = (float(e2e["value"]), hib)
    for k, v in (rep.get("extra") or {}).items():
        if isinstance(v, (int, float)) and not isinstance(v, bool):
            out[k] = (float(v), not k.endswith(("_ms", "_us", "_s", "_latency")))
    return out


def compare(champion: dict, candidate: dict, tolerance: float = 0.03) -> dict:
    a, b = metrics_of(champion), metrics_of(candidate)
    rows, ok = [], True
    for name in a:
        if name not in b:
            rows.append({"metric": name, "missing_in_candidate": True})
            ok = False
            continue
        (va, hib), (vb, _) = a[name], b[name]
        ratio = 1.0 if va == vb else ((vb / va if hib else va / vb) if va and vb else 0.0)      # > 1 = candidate better
        passed = ratio >= 1.0 - tolerance
        ok &= passed
        rows.append({"metric": name, "champion": va, "candidate": vb, "ratio": round(ratio, 4), "higher_is_better": hib, "pass": passed})
    return {"pass": ok and bool(rows), "tolerance": tolerance, "metrics": rows}


def config_diff(a: dict, b: dict, prefix: str = "") -> List[Tuple[str, Any, Any]]:
    out: List[Tuple[str, Any, Any]] = []
    for k in sorted(set(a) | set(b)):
        p = f"{prefix}.{k}" if prefix else k
        x, y = a.get(k), b.get(k)
        if isinstance(x, dict) and isinstance(y, dict):
            out.extend(config_diff(x, y, p))
        elif x != y:
            out.append((p, x, y))
    return out


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("champion")
    ap.add_argument("candidate")
    ap.add_argument("--tolerance", type=float, default=0.03)
    ap.add_argument("--champion-config")
    ap.add_argument("--candidate-config")
    a = ap.parse_args(argv)
    rep = compare(_last_json_line(a.champion), _last_json_line(a.candidate), a.tolerance)
    if a.champion_config and a.candidate_config:
        rep["config_diff"] = [{"path": p, "champion": x, "candidate": y}
                              for p, x, y in config_diff(json.load(open(a.champion_config)), json.load(open(a.candidate_config)))
                              if not p.startswith("autoconfig.")]
    print(json.dumps(rep, indent=1))
    return 0 if rep["pass"] else 1


if __name__ == "__main__":
    sys.exit(main())
