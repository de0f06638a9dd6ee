"""The auto-run pipeline: one command from a model path to a measured, derived configuration.

    python -m layerstorm_b200.cli.autoconfigure --model <weights or shape> --auto-run [--out-dir DIR] [--reset]
        [--calibration FILE] [--trained FILE] [--placement-table FILE] [--train-gen 100]

  step 1  CALIBRATE  measure this machine's loader constants (``runtime/calibration.py``: host->device rate of an expert slot,
                     grouped expert-FFN cost curve), or reuse an artifact whose fingerprint matches this machine and model;
  step 2  DERIVE     solve the configuration against the measured hardware and the model's own shape (``autoconfig/solver.py``);
  step 3  TRAIN      run a short REAL decode under the derived configuration with the loader's traces on
                     (``autoconfig/benchmark.py`` with ``LS_FETCH_TRACE`` / ``LS_ROUTING_TRACE``) and correct the copy constants
                     against it (``utils/loader_xray.py fit-constants``); derive again with the trained constants;
  step 4  PLACE      fit the per-(layer, expert) demand-fetch table from step 3's own routing trace
                     (``utils/loader_xray.py freq-table``) and carry it in ``memory.arena_placement.freq_table``.
The order is forced: the trainer corrects a BASELINE calibration, so that exists first; the training decode needs a bootable
configuration, so derivation precedes it; the placement fit consumes the trace that decode leaves, so it costs no extra boot.  Steps 3
and 4 only run when the derived configuration streams experts (``vram_expert_ratio`` < 1): with every expert resident there is no loader
to train.  Artifacts that exist and match (fingerprint of hardware + model shape) are reused; ``reset`` recomputes them; explicit
paths supply them (which also lets a machine without GPU time re-derive from artifacts it already has).

The GPU-touching steps are behind ``Runners`` (calibrate, training decode): the command line wires the real ones, tests pass fakes.
Every run leaves ``<stem>.autorun.json`` (what ran, what was reused, where the artifacts are) beside the configuration.
Reference: python/autoconfig/pipeline.py (calibrate -> derive -> train -> place, reuse policy, artifact paths), enginerun.py.
"""
from __future__ import annotations

import dataclasses
import hashlib
import json
import os
import subprocess
import sys
from typing import Callable, Dict, List, Optional

from ..models.config import ModelConfig
from .calibration import apply_calibration
from .hwdetect import HardwareInfo
from .solver import Levers, solve, write_result


def artifact_fingerprint(hw: HardwareInfo, shape: ModelConfig) -> str:
    """What a measured artifact is valid for: this machine's hardware fingerprint and the model's expert geometry."""
    key = f"{hw.fingerprint()}|{shape.name}|{shape.hidden}|{shape.moe_inter}|{shape.n_routed}|{shape.n_layers}|{shape.expert_quant}"
    return hashlib.sha256(key.encode()).hexdigest()[:16]


@dataclasses.dataclass
class AutoRunOptions:
    model: str
    out_dir: str = "."
    name: Optional[str] = None
    reset: bool = False
    calibration: Optional[str] = None          # explicit artifacts (reused as they are)
    trained: Optional[str] = None
    placement_table: Optional[str] = None
    train_prompt: int = 512
    train_gen: int = 100
    serve_flags: List[str] = dataclasses.field(default_factory=list)     # passed to the training decode's server boot (e.g. --random-weights)
    draft_bytes: int = 0                        # what a block draft takes on its GPU (the solver keeps it when it fits)


@dataclasses.dataclass
class Runners:
    """The steps that touch the GPU.  ``calibrate(path) -> dict`` writes and returns a calibration document;
    ``training_decode(config_path, fetch_trace, routing_trace, log_path) -> dict`` boots the configuration, decodes and returns the
    benchmark report (the traces are written as a side effect)."""
    calibrate: Callable[[str], dict]
    training_decode: Callable[[str, str, str, str], dict]


def default_runners(opts: AutoRunOptions) -> Runners:
    def calibrate(path: str) -> dict:
        from ..runtime.calibration import calibrate as cal
        return cal(None, "quick", path)

    def training_decode(config_path: str, fetch_trace: str, routing_trace: str, log_path: str) -> dict:
        env = dict(os.environ, LS_FETCH_TRACE=fetch_trace, LS_ROUTING_TRACE=routing_trace)
        cmd = [sys.executable, "-m", "layerstorm_b200.autoconfig.benchmark", "--prompt-len", str(opts.train_prompt), "--gen", str(opts.train_gen),
               "--requests", "1", "--", "--config", config_path, "--model", opts.model, *opts.serve_flags]
        with open(log_path, "w") as log:
            p = subprocess.run(cmd, env=env, stdout=subprocess.PIPE, stderr=log, text=True)
        if p.returncode != 0:
            raise RuntimeError(f"training decode exited {p.returncode}; see {log_path}")
        line = [l for l in p.stdout.splitlines() if l.strip().startswith("{")]
        return json.loads(line[-1]) if line else {}
    return Runners(calibrate, training_decode)


def _load_if_matching(path: str, fp: str, reset: bool) -> Optional[dict]:
    """A stored artifact, if it was measured for this machine and model (and no reset was asked for)."""
    if reset or not path or not os.path.exists(path):
        return None
    try:
        doc = json.load(open(path))
    except (OSError, ValueError):
        return None
    return doc if doc.get("fingerprint") == fp else None


def run_pipeline(shape: ModelConfig, hw: HardwareInfo, levers: Levers, pins: dict, base: Optional[dict], opts: AutoRunOptions,
                 runners: Optional[Runners] = None) -> dict:
    runners = runners or default_runners(opts)
    out_dir = os.path.abspath(opts.out_dir)
    os.makedirs(out_dir, exist_ok=True)
    stem = opts.name or ("auto-" + shape.name.lower().replace(" ", "-"))
    fp = artifact_fingerprint(hw, shape)
    paths = {"config": os.path.join(out_dir, stem + ".autoconfig.json"), "autorun": os.path.join(out_dir, stem + ".autorun.json"),
             "calibration": os.path.abspath(opts.calibration) if opts.calibration else os.path.join(out_dir, f"gpu_loader_calibration_{stem}.json"),
             "trained": os.path.abspath(opts.trained) if opts.trained else os.path.join(out_dir, f"gpu_loader_calibration_{stem}_trained.json"),
             "placement": os.path.abspath(opts.placement_table) if opts.placement_table else os.path.join(out_dir, f"arena_placement_{stem}.csv"),
             "logs": os.path.join(out_dir, stem + ".autorun-logs")}
    os.makedirs(paths["logs"], exist_ok=True)
    record: Dict = {"fingerprint": fp, "model": opts.model, "steps": [], "artifacts": paths}

    def explicit(path: Optional[str]) -> Optional[dict]:
        if not path:
            return None
        doc = json.load(open(path))
        doc["_explicit"] = True
        return doc

    # ---- step 1: calibrate (or reuse)
    cal = explicit(opts.calibration) or _load_if_matching(paths["calibration"], fp, opts.reset)
    if cal is None:
        cal = dict(runners.calibrate(paths["calibration"]) or {})
        cal["fingerprint"] = fp
        json.dump(cal, open(paths["calibration"], "w"), indent=1)
        record["steps"].append({"step": "calibrate", "ran": True, "artifact": paths["calibration"]})
    else:
        record["steps"].append({"step": "calibrate", "ran": False, "reused": paths["calibration"]})

    def derive(constants: dict, placement: str = ""):
        hw2, notes = apply_calibration(hw, constants)
        b = json.loads(json.dumps(base)) if base else {}
        b.setdefault("gpu_loader", {}).update({"enabled": True, "calibration_mode": "loaded", "calibration_path": constants.get("_path", "")})
        if placement:
            b.setdefault("memory", {}).setdefault("arena_placement", {})["freq_table"] = placement
        return solve(shape, hw2, levers, pins, b, draft_bytes=opts.draft_bytes), notes

    # ---- step 2: derive
    cal["_path"] = paths["calibration"]
    res, notes = derive(cal)
    record["steps"].append({"step": "derive", "ran": True, "calibration_notes": notes, "vram_expert_ratio": round(res.candidate.report.vram_expert_ratio, 4)})
    streams = res.candidate.report.vram_expert_ratio < 1.0

    # ---- steps 3 and 4: train the copy constants on a real decode, fit the placement table from its routing
    if not streams:
        record["steps"].append({"step": "train", "ran": False, "why": "every expert is resident: there is no loader to train"})
        record["steps"].append({"step": "place", "ran": False, "why": "every expert is resident"})
    else:
        trained = explicit(opts.trained) or _load_if_matching(paths["trained"], fp, opts.reset)
        placement_ok = bool(opts.placement_table) or (not opts.reset and os.path.exists(paths["placement"]) and trained is not None)
        if trained is None or not placement_ok:
            from ..utils import loader_xray as lx
            from ..utils.cache_sim import read_trace
            write_result(res, paths["config"])                          # the training decode boots this
            ftrace, rtrace = os.path.join(paths["logs"], "fetch_trace.txt"), os.path.join(paths["logs"], "routing_trace.txt")
            for f in (ftrace, rtrace):
                if os.path.exists(f):
                    os.remove(f)
            bench = runners.training_decode(paths["config"], ftrace, rtrace, os.path.join(paths["logs"], "training_decode.log"))
            if trained is None:
                fit = lx.fit_constants(lx.read_fetch_trace(ftrace), calib_gbs=apply_calibration(hw, cal)[0].h2d_gbs)
                trained = {"fingerprint": fp, "version": cal.get("version"), "h2d_gbs": fit["h2d_gb_s"], "batch_overhead_us": fit["batch_overhead_us"],
                           "fit": fit, "baseline": paths["calibration"], "training_decode": {k: bench.get(k) for k in ("value", "unit", "prefill_tok_s") if k in bench}}
                for k in ("devices", "banks"):
                    if k in cal:
                        trained[k] = cal[k]
                json.dump(trained, open(paths["trained"], "w"), indent=1)
                record["steps"].append({"step": "train", "ran": True, "artifact": paths["trained"], "h2d_gb_s": fit["h2d_gb_s"], "r2": fit["r2"]})
            else:
                record["steps"].append({"step": "train", "ran": False, "reused": paths["trained"]})
            if not opts.placement_table:
                slots = max(1, int(res.candidate.report.expert_slots_per_layer))
                counts = lx.fetch_counts([read_trace(rtrace)], slots)
                lx.write_freq_table(paths["placement"], counts, f"auto-run of {opts.model}, {slots} slots per layer")
                record["steps"].append({"step": "place", "ran": True, "artifact": paths["placement"], "keys": len(counts),
                                        "concentration": lx.concentration(counts)})
            else:
                record["steps"].append({"step": "place", "ran": False, "reused": paths["placement"]})
        else:
            record["steps"].append({"step": "train", "ran": False, "reused": paths["trained"]})
            record["steps"].append({"step": "place", "ran": False, "reused": paths["placement"]})
        trained["_path"] = paths["trained"]
        res, notes = derive(trained, paths["placement"])
        record["steps"].append({"step": "derive", "ran": True, "with": "trained constants + placement table", "calibration_notes": notes})

    cfg_path, side = write_result(res, paths["config"])
    record["config"], record["explain"] = cfg_path, side
    json.dump(record, open(paths["autorun"], "w"), indent=1)
    return record
