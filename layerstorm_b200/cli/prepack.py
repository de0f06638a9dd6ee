"""``python -m layerstorm_b200.cli.prepack --model <checkpoint> --out <dir> [--quant nvfp4]`` - write the prepacked expert
store (one slot image per expert + manifest) for a checkpoint.  Resumable: existing files that match are skipped.
Reference: the prepack tool of the reference (tools/prepack_experts, pybind ``prepack_experts``)."""
from __future__ import annotations

import argparse
import sys
from typing import Optional

from ..formats.prepacked import PrepackedSource, prepack_model
from ..models.checkpoint import open_checkpoint


def main(argv: Optional[list[str]] = None) -> int:
    ap = argparse.ArgumentParser(prog="layerstorm_b200.cli.prepack")
    ap.add_argument("--model", required=True, help="HF safetensors directory or .gguf file")
    ap.add_argument("--out", required=True)
    ap.add_argument("--quant", default=None, choices=["bf16", "fp8_e4m3", "nvfp4", "gguf_q4_k"])
    ap.add_argument("--verify", action="store_true", help="re-read every file and check its digest")
    a = ap.parse_args(argv)
    cfg, ck = open_checkpoint(a.model)
    wr = prepack_model(cfg, ck, a.out, a.quant)
    print(f"prepacked {wr.written} experts ({wr.skipped} unchanged) -> {a.out}  [{wr.quant}, {wr.ef.stride} bytes per slot]")
    if a.verify:
        n, bad = PrepackedSource(a.out).verify_all()
        print(f"verified {n} files, {bad} bad")
        return 1 if bad else 0
    return 0


if __name__ == "__main__":
    sys.exit(main())
