"""Autoconfig: derive a complete engine configuration from (model, machine, a few levers).

Levers   vram_expert_ratio            fraction of each GPU's owned experts that must be resident in HBM
         total_active_context_tokens  max_concurrent_requests x max_sequence_length; the solver owns the split
         prefer  speed|balanced|capacity   a sort key over one candidate lattice - never a weight, so it can never
                                           cause a refusal that another preference would avoid
         accuracy compact|standard|high|superior   floor on the attention-backend ladder
Pins     ``path=value`` hard constraints; each removes an axis from the lattice, and a refusal names the pin
         that made the problem infeasible.
Ladder   P1 order GPUs -> P2 tensor-parallel degree -> P3 roles -> P4 KV mode -> P5 indexer mode -> K1 context
         split -> K2 sizing -> K3 tiering -> E1 searched fit over the lattice -> P6 draft -> H1 host arena /
         NUMA -> M1 mechanical knobs.  Every step appends to an explain record that is written beside the
         config as ``<output>.explain.json``.
Reference: docs/AUTOCONFIG_MODEL.md:128-311,395-499 (levers, pins, ladder, refusal wording) and
python/autoconfig/*.  The machine model differs: identical GPUs on one NVSwitch domain make tensor
parallelism and expert parallelism cheap, so most of the reference's PCIe-priced axes collapse.
"""
from __future__ import annotations

import copy
import json
from dataclasses import dataclass, field
from typing import Any

from ..config.loader import ConfigError, deep_merge, get_path, load_config, model_section_from, set_path, validate
from ..models.config import ModelConfig
from . import sizing, templates
from .hwdetect import HardwareInfo

PINNABLE = (
    "parallelism.tensor_parallelism", "hardware.dcp_kv_mode", "hardware.dcp_indexer_mode", "compute.attention_backend",
    "serving.max_concurrent_requests", "serving.max_sequence_length", "speculation.method", "memory.kv_tiering.enabled",
    "memory.kv_cache.page_size_tokens", "orchestrator.prefill_chunk_tokens", "quantization.kv_cache",
)


class AutoconfigRefusal(RuntimeError):
    """No configuration satisfies the constraints; ``binding`` names what to relax."""

    def __init__(self, msg: str, binding: str, explain: dict):
        super().__init__(msg)
        self.binding = binding
        self.explain = explain


@dataclass
class Levers:
    vram_expert_ratio: float | None = None
    total_active_context_tokens: int | None = None
    prefer: str = "balanced"
    accuracy: str = "standard"


@dataclass
class Candidate:
    tp: int
    indexer_mode: str
    backend: str
    draft: bool
    concurrency: int
    seq_len: int
    report: sizing.FitReport | None = None

    def key(self):
        return (self.tp, self.indexer_mode, self.backend, self.draft, self.concurrency, self.seq_len)


@dataclass
class Result:
    config: dict
    explain: dict
    candidate: Candidate
    warnings: list[str] = field(default_factory=list)


def _pow2_le(n: int) -> int:
    p = 1
    while p * 2 <= n:
        p *= 2
    return p


def _tp_options(mc: ModelConfig, n_gpus: int) -> list[int]:
    out = []
    p = 1
    while p <= min(8, n_gpus):
        heads_ok = mc.n_heads % p == 0 and (mc.kda_heads % p == 0 if mc.kda_heads else True)
        if heads_ok and n_gpus % p == 0:
            out.append(p)
        p *= 2
    return out or [1]


def _ladder(mc: ModelConfig, accuracy: str) -> list[str]:
    lad = sizing.V4_LADDER if mc.architecture == "deepseek_v4" else sizing.MLA_LADDER
    # the floor is also the choice: a more accurate backend only costs memory, so it is taken only when pinned
    return [lad[sizing.ACCURACY_FLOOR[accuracy]]]


def _modelled_decode_ms(mc: ModelConfig, hw: HardwareInfo, tp: int, n_gpus: int, rep: sizing.FitReport) -> float:
    """Coarse batch-1 decode step time: weight bytes streamed per GPU / HBM bandwidth + per-layer reduction
    latency + expert misses fetched from host."""
    res = sizing.resident_bytes(mc, tp, n_gpus, True)
    act_experts = mc.top_k * mc.n_moe_layers() * sizing.expert_slot_bytes(mc) / n_gpus
    stream = (res.attention + res.dense_ffn + res.shared_expert + res.head + act_experts) / (hw.hbm_gbs * 1e9)
    reduce_lat = 0.0 if n_gpus == 1 else mc.n_layers * 2 * 12e-6
    miss = (1.0 - rep.vram_expert_ratio) * mc.top_k * mc.n_moe_layers() * sizing.expert_slot_bytes(mc) / n_gpus / (hw.h2d_gbs * 1e9)
    fixed = mc.n_layers * 12 * 2.5e-6
    return (stream + reduce_lat + miss + fixed) * 1e3


def solve(mc: ModelConfig, hw: HardwareInfo, levers: Levers | None = None, pins: dict[str, Any] | None = None,
          base: dict | None = None, draft_bytes: int = 0) -> Result:
    levers = levers or Levers()
    pins = dict(pins or {})
    ex: dict[str, Any] = {"levers": levers.__dict__.copy(), "pins": pins, "steps": [], "fingerprint": hw.fingerprint()}

    def step(name, decision, why):
        ex["steps"].append({"step": name, "decision": decision, "why": why})

    for p in pins:
        if p not in PINNABLE:
            raise AutoconfigRefusal(f"'{p}' is not a pinnable field; pinnable: {', '.join(PINNABLE)}", p, ex)
    if levers.prefer not in ("speed", "balanced", "capacity"):
        raise AutoconfigRefusal(f"prefer '{levers.prefer}' is not one of speed, balanced, capacity", "prefer", ex)
    if levers.accuracy not in sizing.ACCURACY_FLOOR:
        raise AutoconfigRefusal(f"accuracy '{levers.accuracy}' is not one of compact, standard, high, superior", "accuracy", ex)
    if not hw.gpus:
        raise AutoconfigRefusal("no GPU was detected; autoconfig needs at least one", "hardware.gpus", ex)

    # P1: order GPUs - largest memory first, then by id; identical GPUs keep their bus order
    gpus = sorted(hw.gpus, key=lambda g: (-round(g.vram_gb), g.id))
    top = [g for g in gpus if round(g.vram_gb) == round(gpus[0].vram_gb) and g.type == gpus[0].type]
    n = len(top)
    step("P1", {"order": [g.id for g in gpus], "top_class": gpus[0].type, "count": n},
         "GPUs of the largest class carry the model; smaller ones are left to the draft model")
    vram = min(g.vram_gb for g in top)

    # P2: tensor-parallel degrees to search
    tps = _tp_options(mc, n)
    if "parallelism.tensor_parallelism" in pins:
        t = pins["parallelism.tensor_parallelism"]
        if t not in tps:
            raise AutoconfigRefusal(f"pin parallelism.tensor_parallelism={t} is not feasible: it must be a power of two that divides "
                                    f"{mc.n_heads} heads and {n} GPUs (options {tps})", "parallelism.tensor_parallelism", ex)
        tps = [t]
    step("P2", {"tp_options": tps}, f"powers of two dividing {mc.n_heads} heads" + (f" / {mc.kda_heads} KDA heads" if mc.kda_heads else "") + f" and {n} GPUs")

    # accuracy ladder
    ladder = _ladder(mc, levers.accuracy)
    if "compute.attention_backend" in pins:
        b = pins["compute.attention_backend"]
        full = sizing.V4_LADDER if mc.architecture == "deepseek_v4" else sizing.MLA_LADDER
        if b not in full:
            raise AutoconfigRefusal(f"pin compute.attention_backend={b} is not a backend of architecture {mc.architecture}", "compute.attention_backend", ex)
        if full.index(b) < sizing.ACCURACY_FLOOR[levers.accuracy]:
            raise AutoconfigRefusal(f"pin compute.attention_backend={b} is below the accuracy floor '{levers.accuracy}'", "compute.attention_backend", ex)
        ladder = [b]
    if levers.accuracy == "superior" and "compute.attention_backend" not in pins:
        # defined, but priced out of the default search: unquantised KV rows double the cache
        step("A", {"ladder": ladder}, "accuracy 'superior' keeps bf16 KV rows (2x the FP8 cache)")

    # K1: context budget
    sec = (base or {}).get("serving", {})
    conc0 = pins.get("serving.max_concurrent_requests", sec.get("max_concurrent_requests", 32))
    len0 = pins.get("serving.max_sequence_length", sec.get("max_sequence_length", min(mc.max_position, 131072)))
    if levers.total_active_context_tokens:
        tot = int(levers.total_active_context_tokens)
        if "serving.max_sequence_length" in pins and "serving.max_concurrent_requests" not in pins:
            conc0 = max(1, tot // len0)
        elif "serving.max_concurrent_requests" in pins and "serving.max_sequence_length" not in pins:
            len0 = max(1, tot // conc0)
        elif "serving.max_concurrent_requests" not in pins:
            len0 = min(len0, tot)
            conc0 = max(1, tot // len0)
    step("K1", {"max_concurrent_requests": conc0, "max_sequence_length": len0},
         "total_active_context_tokens = concurrency x length; concurrency is degraded first, then length")

    want_draft = pins.get("speculation.method", "dspark" if draft_bytes else "none") not in ("none", "null")
    idx_modes = ["replicated", "local"] if mc.has_indexer else ["replicated"]
    if "hardware.dcp_indexer_mode" in pins:
        idx_modes = [pins["hardware.dcp_indexer_mode"]]
    base_chunk = (base or {}).get("orchestrator", {}).get("prefill_chunk_tokens")
    chunk = pins.get("orchestrator.prefill_chunk_tokens", base_chunk or templates.prefill_chunk_for(conc0))
    min_ratio = levers.vram_expert_ratio or 0.0

    # E1: the lattice, in relaxation order
    def relaxations():
        conc, ln = conc0, len0
        seen = set()
        while True:
            for dr in ([True, False] if want_draft and "speculation.method" not in pins else [want_draft]):
                if (conc, ln, dr) not in seen:
                    seen.add((conc, ln, dr))
                    yield conc, ln, dr
            if conc > 1 and "serving.max_concurrent_requests" not in pins:
                conc = max(1, conc // 2)
            elif ln > 4096 and "serving.max_sequence_length" not in pins:
                ln //= 2
            else:
                return

    feasible: list[Candidate] = []
    tried = 0
    last_binding = ""
    for conc, ln, dr in relaxations():
        level: list[Candidate] = []
        for tp in tps:
            kv_mode = pins.get("hardware.dcp_kv_mode", "sharded" if tp > 1 else "replicated")
            for im in idx_modes:
                for be in ladder:
                    tried += 1
                    rep = sizing.fit(mc, vram_gb=vram, n_gpus=n, tp=tp, backend=be, kv_mode=kv_mode, context_tokens=conc * ln,
                                     concurrency=conc, max_rows=max(chunk, conc), draft_bytes=draft_bytes if dr else 0,
                                     embed_on_host=True, min_slot_fraction=min_ratio)
                    c = Candidate(tp, im, be, dr, conc, ln, rep)
                    if rep.ok:
                        level.append(c)
                    else:
                        last_binding = rep.binding
        if level:
            feasible = level
            break
    if not feasible:
        binding = next((p for p in ("serving.max_sequence_length", "serving.max_concurrent_requests", "parallelism.tensor_parallelism",
                                    "compute.attention_backend") if p in pins), "")
        what = f"pin {binding}={pins[binding]}" if binding else (f"vram_expert_ratio={min_ratio}" if min_ratio else last_binding or "the model's resident weights")
        raise AutoconfigRefusal(
            f"no configuration fits {n}x {gpus[0].type} ({vram:.0f} GB): after {tried} candidates the binding constraint is {what}"
            + (f" ({last_binding} does not fit)" if last_binding and binding else ""), binding or what, ex)

    # prefer = sort key over the feasible set of the first level that fits
    def speed_key(c: Candidate):
        return (_modelled_decode_ms(mc, hw, c.tp, n, c.report), -ladder.index(c.backend), c.indexer_mode != "replicated")

    def capacity_key(c: Candidate):
        return (-c.report.expert_slots_per_layer, -(c.report.vram_budget - c.report.resident - c.report.kv), c.tp)

    def balanced_key(c: Candidate):
        return (c.indexer_mode != "replicated", not c.draft, -ladder.index(c.backend), _modelled_decode_ms(mc, hw, c.tp, n, c.report))

    keys = {"speed": speed_key, "capacity": capacity_key, "balanced": balanced_key}
    best = min(feasible, key=keys[levers.prefer])
    others = {k: min(feasible, key=f).key() for k, f in keys.items()}
    prefer_mattered = len(set(others.values())) > 1
    step("E1", {"candidates_tried": tried, "feasible_at_level": len(feasible), "chosen": best.key(),
                "prefer_changed_outcome": prefer_mattered},
         (f"prefer={levers.prefer} chose among {len(feasible)} feasible candidates" if prefer_mattered else
          "every preference picks the same candidate"))
    if (best.concurrency, best.seq_len) != (conc0, len0):
        step("E1.relax", {"max_concurrent_requests": best.concurrency, "max_sequence_length": best.seq_len},
             "the requested context budget did not fit; concurrency was halved before length")
    if want_draft and not best.draft:
        step("P6", {"draft": False}, "the draft model was dropped to make the target fit")

    rep = best.report
    kv_mode = pins.get("hardware.dcp_kv_mode", "sharded" if best.tp > 1 else "replicated")
    # K3: tiering only helps sparse attention with self-contained rows, and only when KV is the tight term
    tiering = bool(pins.get("memory.kv_tiering.enabled", mc.has_indexer and rep.kv > 0.35 * rep.vram_budget))
    step("K3", {"kv_tiering": tiering}, "ON iff sparse attention and the KV cache takes more than 35% of a GPU")

    # H1: host arena for experts that are not resident
    host_need_gb = rep.host_expert_bytes * n / sizing.GiB
    host_ok = host_need_gb <= hw.system_ram_gb * 0.9 if hw.system_ram_gb else True
    if not host_ok:
        raise AutoconfigRefusal(f"the experts that do not fit in HBM need {host_need_gb:.0f} GB of pinned host memory but the machine has "
                                f"{hw.system_ram_gb:.0f} GB", "hardware.system_ram_gb", ex)
    step("H1", {"host_expert_gb": round(host_need_gb, 1), "numa_nodes": hw.numa_nodes},
         "experts beyond the HBM slots live in a pinned arena, interleaved over NUMA nodes by GPU affinity")

    # P3 + M1: write the config
    cfg = load_config(base, check=False) if base is not None else load_config(None, check=False)
    cfg["model"] = deep_merge(cfg["model"], model_section_from(mc))
    roles = {g.id: ["attention", "resident", "expert_streaming"] for g in top}
    for g in gpus:
        if g.id not in roles:
            roles[g.id] = ["draft"] if best.draft else []
    cfg["hardware"] = deep_merge(cfg["hardware"], hw.hardware_section(roles))
    cfg["hardware"]["tp_array"] = [g.id for g in top[:best.tp]]
    cfg["hardware"]["dcp_kv_mode"] = kv_mode
    cfg["hardware"]["dcp_indexer_mode"] = best.indexer_mode
    cfg["hardware"]["dcp_enabled"] = best.tp > 1
    cfg["parallelism"]["tensor_parallelism"] = best.tp
    cfg["parallelism"]["expert_parallelism"] = n
    be = best.backend
    cfg["compute"]["attention_backend"] = "snapmla" if be == "bf16_mla" else be
    cfg["quantization"]["kv_cache"] = {"turboquant_mla": "turboquant4", "csa_hca_tq": "turboquant4", "bf16_mla": "bf16", "csa_hca": "bf16"}.get(be, "fp8_e4m3")
    cfg["quantization"]["weights"] = mc.expert_quant if mc.expert_quant in sizing.QUANT_BITS else "nvfp4"
    cfg["serving"]["max_concurrent_requests"] = best.concurrency
    cfg["serving"]["max_sequence_length"] = best.seq_len
    cfg["orchestrator"]["max_batch_size"] = max(1, min(cfg["orchestrator"]["max_batch_size"], best.concurrency))
    cfg["orchestrator"]["prefill_chunk_tokens"] = chunk
    cfg["memory"]["kv_tiering"]["enabled"] = tiering
    page = pins.get("memory.kv_cache.page_size_tokens", 64)
    cfg["memory"]["kv_cache"]["page_size_tokens"] = page
    cfg["memory"]["kv_cache"]["max_pages_per_gpu"] = int(-(-best.concurrency * best.seq_len // page) + best.concurrency)
    cfg["memory"]["pin_host_expert_pool"] = rep.host_expert_bytes > 0
    cfg["speculation"]["method"] = pins.get("speculation.method", "dspark") if best.draft else "none"
    cfg["speculation"]["enabled"] = best.draft
    cfg["autoconfig"].update({"enabled": True, "vram_expert_ratio": round(rep.vram_expert_ratio, 4),
                              "total_active_context_tokens": best.concurrency * best.seq_len, "prefer": levers.prefer,
                              "accuracy": levers.accuracy, "fingerprint": hw.fingerprint()})
    # T1: family template for what neither geometry nor hardware decides; the base configuration and pins win
    user_set = {p for p, _ in templates._leaves(base or {})} | set(pins)
    copied = templates.apply_template(cfg, mc.architecture, user_set)
    step("T1", {"family": templates.family_of(mc.architecture), "copied": copied}, "family template (kind = template); base configuration and pins win")
    for p, v in pins.items():
        set_path(cfg, p, v)
    step("M1", {"expert_slots_per_layer_per_gpu": rep.expert_slots_per_layer, "owned_experts_per_gpu": rep.expert_slots_wanted,
                "bytes": {"budget": rep.vram_budget, "resident": rep.resident, "kv": rep.kv, "recurrent": rep.recurrent,
                          "workspace": rep.workspace, "draft": rep.draft}},
         "mechanical knobs follow from the chosen candidate")
    ex["modelled_decode_ms"] = round(_modelled_decode_ms(mc, hw, best.tp, n, rep), 3)
    warnings = []
    if rep.vram_expert_ratio < 1.0:
        warnings.append(f"{rep.expert_slots_per_layer}/{rep.expert_slots_wanted} of each GPU's experts are resident; the rest stream from host memory")
    try:
        validate(cfg)
    except ConfigError as e:           # a pin combination the validator rejects
        raise AutoconfigRefusal(str(e), e.problems[0].split(":")[0], ex)
    return Result(cfg, ex, best, warnings)


def write_result(res: Result, output_path: str) -> tuple[str, str]:
    """Write the config and its explain sidecar; returns both paths."""
    with open(output_path, "w") as fh:
        json.dump(res.config, fh, indent=1)
    side = output_path + ".explain.json"
    with open(side, "w") as fh:
        json.dump({"explain": res.explain, "warnings": res.warnings}, fh, indent=1)
    return output_path, side


def explain_text(res: Result) -> str:
    lines = [f"autoconfig ({res.explain['fingerprint']}): tp={res.candidate.tp} backend={res.candidate.backend} "
             f"concurrency={res.candidate.concurrency} x length={res.candidate.seq_len} draft={'on' if res.candidate.draft else 'off'}"]
    for s in res.explain["steps"]:
        lines.append(f"  [{s['step']}] {s['why']}: {json.dumps(s['decision'], default=str)}")
    lines += [f"  warning: {w}" for w in res.warnings]
    return "\n".join(lines)
