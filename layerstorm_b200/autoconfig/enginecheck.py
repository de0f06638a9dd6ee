"""Cross-check of the solver's model of the engine against what a booted engine really allocated.

The solver sizes a configuration from formulas (``autoconfig/sizing.py``): bytes of a KV row, of an expert slot, of a sequence's
recurrent state, of the resident weights.  The engine computes the same quantities when it allocates.  When the two drift apart
nothing notices until a derived configuration fails to boot or refuses a request it should take - so the check is a TABLE of
(solver figure, engine figure, tolerance, exact-or-bound) rows, run against ``Engine.vram_plan`` and the model's own tensors after
every boot that wants it; a new quantity is a new row, not new code.

Honesty rule: an EXACT row that diverges beyond its tolerance fails.  A BOUND row states a direction (the solver must not
UNDER-estimate memory): diverging in the allowed direction is a warning, the other way a failure - a violated bound is the dangerous
case.  A row whose figure cannot be computed for this model is reported UNCHECKED; silence never reads as agreement.

    python -m layerstorm_b200.autoconfig.enginecheck --model tiny-mla-moe --random-weights     # boots, checks, prints the table
Reference: python/autoconfig/enginecheck.py (CHECKS table of solver site vs engine boot-log site, exact / bound semantics).
"""
from __future__ import annotations

import dataclasses
import json
import sys
from typing import Callable, List, Optional

from ..models.config import ModelConfig
from . import sizing


@dataclasses.dataclass
class CheckRow:
    name: str
    unit: str
    kind: str                                   # "exact" | "upper_bound" (solver >= engine is fine, solver < engine fails)
    tolerance: float                            # relative
    solve: Callable[[ModelConfig, dict], Optional[float]]
    observe: Callable[[object], Optional[float]]


@dataclasses.dataclass
class CheckResult:
    name: str
    unit: str
    kind: str
    solver: Optional[float]
    engine: Optional[float]
    status: str                                 # ok | warning | FAIL | unchecked
    note: str = ""


def _kv_backend(engine) -> str:
    return {"fp8": "snapmla", "bf16": "bf16_mla", "tq4": "turboquant_mla"}[engine.model.kv_fmt]


def _solve_kv(mc, ctx):
    return float(sizing.kv_bytes_per_token(mc, ctx["backend"], 1, "replicated"))


def _obs_kv(engine):
    return float(engine.model.cache_bytes_per_token())


def _solve_slot(mc, ctx):
    return float(sizing.expert_slot_bytes(mc, ctx["expert_quant"])) if mc.n_routed else None


def _obs_slot(engine):
    a = [L["arena"] for L in engine.model.layers if L.get("arena") is not None]
    return float(a[0].ef.stride) if a else None


def _solve_rec(mc, ctx):
    v = sizing.recurrent_state_bytes_per_seq(mc, ctx["tp"])
    return float(v) if v else None


def _obs_rec(engine):
    m = engine.model
    v = sum(t[0].numel() * t.element_size() for t in list(m.kda_state.values()) + list(m.kda_conv.values()))
    return float(v) if v else None


def _solve_resident(mc, ctx):
    rb = sizing.resident_bytes(mc, ctx["tp"], ctx["tp"], ctx["embed_on_host"])
    return float(rb.total - rb.shared_expert)          # the engine keeps shared experts in the expert arena, not with the resident weights


def _obs_resident(engine):
    m = engine.model
    arenas = [L["arena"] for L in m.layers if L.get("arena") is not None]
    return float(m.weight_bytes() - sum(a.data.numel() for a in arenas))


def _solve_pages(mc, ctx):
    return float(ctx["max_seqs"] * ((ctx["max_ctx"] + ctx["page"] - 1) // ctx["page"])) if ctx.get("pages_auto") else None


def _obs_pages(engine):
    return float(engine.num_pages)


CHECKS: List[CheckRow] = [
    CheckRow("kv_bytes_per_token", "B", "exact", 0.0, _solve_kv, _obs_kv),
    CheckRow("expert_slot_bytes", "B", "upper_bound", 0.08, _solve_slot, _obs_slot),
    CheckRow("recurrent_state_bytes_per_sequence", "B", "exact", 0.0, _solve_rec, _obs_rec),
    CheckRow("resident_weight_bytes", "B", "upper_bound", 0.15, _solve_resident, _obs_resident),
    CheckRow("kv_pages", "pages", "exact", 0.0, _solve_pages, _obs_pages),
]


def context_of(engine, pages_auto: bool = True) -> dict:
    m = engine.model
    arenas = [L["arena"] for L in m.layers if L.get("arena") is not None]
    from ..models.device_model import _FMT_NAME
    eq = _FMT_NAME[arenas[0].ef.fmt] if arenas else m.cfg.expert_quant
    return {"backend": _kv_backend(engine), "tp": m.tp_size, "expert_quant": eq, "embed_on_host": not m.embed.is_cuda, "max_seqs": engine.max_seqs,
            "max_ctx": engine.max_ctx, "page": engine.page, "pages_auto": pages_auto}


def run_checks(engine, ctx: Optional[dict] = None, rows: Optional[List[CheckRow]] = None) -> List[CheckResult]:
    ctx = context_of(engine) if ctx is None else ctx
    out = []
    for r in rows or CHECKS:
        try:
            s, e = r.solve(engine.cfg, ctx), r.observe(engine)
        except Exception as ex:                 # noqa: BLE001 - a row that cannot be computed is reported, not raised
            out.append(CheckResult(r.name, r.unit, r.kind, None, None, "unchecked", f"{type(ex).__name__}: {ex}"))
            continue
        if s is None or e is None:
            out.append(CheckResult(r.name, r.unit, r.kind, s, e, "unchecked", "not applicable to this model"))
            continue
        rel = (s - e) / max(abs(e), 1e-9)
        if abs(rel) <= max(r.tolerance if r.kind == "exact" else 0.0, 1e-12):
            st, note = "ok", ""
        elif r.kind == "exact":
            st, note = "FAIL", f"solver {rel:+.1%} against the engine (exact row)"
        elif rel >= 0:
            st = "ok" if rel <= r.tolerance else "warning"
            note = f"solver over-estimates by {rel:.1%}" + ("" if st == "ok" else f" (more than {r.tolerance:.0%}: capacity is left unused)")
        else:
            st, note = "FAIL", f"solver UNDER-estimates by {-rel:.1%}: a derived configuration can overcommit the GPU"
        out.append(CheckResult(r.name, r.unit, r.kind, s, e, st, note))
    return out


def render(results: List[CheckResult]) -> str:
    lines = [f"{'quantity':38s} {'kind':12s} {'solver':>16s} {'engine':>16s}  status"]
    for r in results:
        f = lambda v: "-" if v is None else f"{v:,.0f}"
        lines.append(f"{r.name:38s} {r.kind:12s} {f(r.solver):>16s} {f(r.engine):>16s}  {r.status}{'  ' + r.note if r.note else ''}")
    return "\n".join(lines)


def main(argv=None) -> int:
    """Boot the engine exactly as ``serve`` would (same flags), run the table, exit 1 on a failed row."""
    from ..cli import serve
    args = serve.build_parser().parse_args(argv)
    cfg, shape, ckpt, _ = serve.resolve_config(args)
    eng = serve.build_engine(cfg, shape, ckpt, args)
    pages = cfg["memory"]["kv_cache"]["max_pages_per_gpu"]
    res = run_checks(eng, context_of(eng, pages_auto=pages in ("auto", None)))
    print(render(res))
    print(json.dumps([dataclasses.asdict(r) for r in res]))
    return 1 if any(r.status == "FAIL" for r in res) else 0


if __name__ == "__main__":
    sys.exit(main())
