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
    p.add_argument("--print", dest="show", action="store_true", help="print the explanation")
    p.add_argument("--probe-only", action="store_true", help="print what the model path is (format, shape, quantisation, size) and exit")
    return p


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
        if args.auto_run:
            from ..autoconfig.pipeline import AutoRunOptions, run_pipeline
            rec = run_pipeline(shape, hw, Levers(args.vram_expert_ratio, args.total_active_context_tokens, args.prefer, args.accuracy),
                               collect_pins(args.pin), base,
                               AutoRunOptions(model=args.model, out_dir=args.out_dir, reset=args.reset, calibration=args.calibration, trained=args.trained,
                                              placement_table=args.placement_table, train_gen=args.train_gen, serve_flags=args.serve_flag))
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
                    collect_pins(args.pin), base)
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
