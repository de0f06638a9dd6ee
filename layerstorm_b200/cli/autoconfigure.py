"""``python -m layerstorm_b200.cli.autoconfigure`` - derive an engine configuration for a model on this
machine (or on a described machine) and write it with its explain sidecar.

Reference: python/cli/autoconfigure.py (same levers, pins and refusal behaviour).
Exit codes: 0 written, 2 bad arguments / config, 3 refused (the message names what to relax).
"""
from __future__ import annotations

import argparse
import json
import sys
from typing import Optional

from ..autoconfig import AutoconfigRefusal, HardwareInfo, Levers, PINNABLE, detect, explain_text, solve, synthetic, write_result
from ..config import ConfigError
from .serve import collect_pins, resolve_model


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="layerstorm_b200.cli.autoconfigure")
    p.add_argument("--model", required=True, help="checkpoint path or built-in shape name")
    p.add_argument("--config", help="base configuration to start from")
    p.add_argument("--output", "-o", default="layerstorm_autoconfig.json")
    p.add_argument("--prefer", choices=["speed", "balanced", "capacity"], default="balanced")
    p.add_argument("--accuracy", choices=["compact", "standard", "high", "superior"], default="standard")
    p.add_argument("--vram-expert-ratio", type=float, default=None)
    p.add_argument("--total-active-context-tokens", type=int, default=None)
    p.add_argument("--pin", action="append", default=[], metavar="PATH=VALUE|FILE.json", help="pinnable: " + ", ".join(PINNABLE))
    p.add_argument("--hardware", help="JSON hardware descriptor to plan for instead of probing this machine")
    p.add_argument("--assume-gpus", type=int, default=None, help="plan for N B200 GPUs (no probe)")
    p.add_argument("--calibration", help="loader calibration or measured-peaks JSON: replaces the default bandwidths of the step-time model")
    p.add_argument("--auto-run", action="store_true",
                   help="the whole pipeline: calibrate this machine (or reuse a matching artifact), derive, train the copy constants on a short "
                        "real decode, fit the expert placement table from it, derive again (autoconfig/pipeline.py)")
    p.add_argument("--out-dir", default=".", help="--auto-run: where the configuration and the measured artifacts go")
    p.add_argument("--reset", action="store_true", help="--auto-run: measure again even where a matching artifact exists")
    p.add_argument("--trained", help="--auto-run: trained loader constants to reuse")
    p.add_argument("--placement-table", help="--auto-run: demand-fetch table to carry instead of fitting one")
    p.add_argument("--train-gen", type=int, default=100, help="--auto-run: tokens of the training decode")
    p.add_argument("--serve-flag", action="append", default=[], help="--auto-run: extra flag of the training decode's server boot (e.g. --random-weights)")
    p.add_argument("--draft-checkpoint", help="a dspark speculator checkpoint (directory with config.json + model.safetensors): the block draft is "
                                             "sized (weights in speculation.dspark.draft_weights_quant + its contexts) and kept when it fits beside the target")
    p.add_argument("--print", dest="show", action="store_true", help="print the explanation")
    p.add_argument("--probe-only", action="store_true", help="print what the model path is (format, shape, quantisation, size) and exit")
    return p


def plan_block_draft(path: str, shape, base: Optional[dict], pins: dict):
    """(base configuration carrying the draft's settings, bytes the draft takes on its GPU) for a dspark speculator checkpoint; the
    checkpoint must have been trained for this target (hidden size, vocabulary, aux layers inside the model)."""
    import os
    from ..speculation import dspark as dsp
    if not dsp.is_dspark_checkpoint(path):
        raise ConfigError([f"--draft-checkpoint: {path} is not a dspark speculator checkpoint (config.json with speculators_model_type = dspark)"])
    try:
        dc = dsp.DsparkCheckpointConfig.from_json(json.load(open(os.path.join(path, "config.json"))))
    except (KeyError, ValueError) as e:
        raise ConfigError([f"--draft-checkpoint: {e}"])
    problems = []
    if dc.hidden_size != shape.hidden or dc.vocab_size != shape.vocab:
        problems.append(f"the draft was trained for hidden {dc.hidden_size} / vocabulary {dc.vocab_size}, the target has {shape.hidden} / {shape.vocab}")
    if any(l < 0 or l > shape.n_layers for l in dc.aux_hidden_state_layer_ids):
        problems.append(f"aux layers {dc.aux_hidden_state_layer_ids} do not fit a target of {shape.n_layers} layers")
    if problems:
        raise ConfigError(["--draft-checkpoint: " + p for p in problems])
    base = json.loads(json.dumps(base)) if base else {}
    ds = base.setdefault("speculation", {}).setdefault("dspark", {})
    ds.update({"checkpoint_path": os.path.abspath(path), "block_size": dc.block_size, "speculative_tokens": dc.speculative_tokens, "markov_rank": dc.markov_rank,
               "mask_token_id": dc.mask_token_id, "draft_vocab_size": dc.draft_vocab_size, "aux_hidden_state_layer_ids": list(dc.aux_hidden_state_layer_ids)})
    ds.setdefault("confidence_enabled", dc.enable_confidence_head)
    quant = pins.get("speculation.dspark.draft_weights_quant", ds.get("draft_weights_quant", "bf16"))
    ctx = int(pins.get("speculation.dspark.draft_context_capacity_tokens", ds.get("draft_context_capacity_tokens", 8192)))
    mem = dsp.draft_memory_bytes(dc, quant, ctx, int(os.environ.get("LSB_DSPARK_CONTEXTS", "4")))
    print(f"block draft: {mem['weights'] / 1e9:.2f} GB of {quant} weights + {mem['contexts'] / 1e9:.2f} GB of draft contexts", file=sys.stderr)
    return base, mem["total"]


def main(argv: Optional[list[str]] = None) -> int:
    args = build_parser().parse_args(argv)
    if args.probe_only:
        from ..autoconfig.modelprobe import probe
        try:
            print(json.dumps(probe(args.model).to_dict(), indent=1))
        except (OSError, ValueError) as e:
            print(f"--model: {e}", file=sys.stderr)
            return 2
        return 0
    try:
        base = json.load(open(args.config)) if args.config else None
        shape, _ = resolve_model(args, base)
        if shape is None:
            raise ConfigError(["--model: no config.json beside the checkpoint; pass a shape name or a full --config"])
        if args.hardware:
            hw = HardwareInfo.from_dict(json.load(open(args.hardware)))
        elif args.assume_gpus:
            hw = synthetic(args.assume_gpus)
        else:
            hw = detect((base or {}).get("hardware", {}).get("nvme_paths"))
        draft_bytes = 0
        if args.draft_checkpoint:
            base, draft_bytes = plan_block_draft(args.draft_checkpoint, shape, base, collect_pins(args.pin))
        if args.auto_run:
            from ..autoconfig.pipeline import AutoRunOptions, run_pipeline
            rec = run_pipeline(shape, hw, Levers(args.vram_expert_ratio, args.total_active_context_tokens, args.prefer, args.accuracy),
                               collect_pins(args.pin), base,
                               AutoRunOptions(model=args.model, out_dir=args.out_dir, reset=args.reset, calibration=args.calibration, trained=args.trained,
                                              placement_table=args.placement_table, train_gen=args.train_gen, serve_flags=args.serve_flag,
                                              draft_bytes=draft_bytes))
            for st in rec["steps"]:
                print("auto-run:", json.dumps(st))
            print(f"wrote {rec['config']} and {rec['artifacts']['autorun']}")
            return 0
        if args.calibration:
            from ..autoconfig.calibration import apply_calibration
            hw, notes = apply_calibration(hw, json.load(open(args.calibration)))
            for n in notes:
                print("calibration:", n, file=sys.stderr)
        res = solve(shape, hw, Levers(args.vram_expert_ratio, args.total_active_context_tokens, args.prefer, args.accuracy),
                    collect_pins(args.pin), base, draft_bytes=draft_bytes)
    except ConfigError as e:
        print(str(e), file=sys.stderr)
        return 2
    except AutoconfigRefusal as e:
        print(f"autoconfig refused: {e}\n  relax: {e.binding}", file=sys.stderr)
        return 3
    cfg_path, side = write_result(res, args.output)
    if args.show:
        print(explain_text(res))
    print(f"wrote {cfg_path} and {side}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
