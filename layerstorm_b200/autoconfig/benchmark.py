"""Benchmark mode: boot a configuration exactly as ``serve.py`` would, measure it, print one JSON report, exit.

Takes the same flags as ``layerstorm_b200.cli.serve`` (``--config`` / ``--autoconfig`` / ``--model`` / ``--random-weights`` /
``--test-engine`` ...) after ``--``, builds the engine and the orchestrator through the server's own boot path (no HTTP), sends one
warm-up request and ``--requests`` measured requests of ``--prompt-len`` synthetic tokens generating ``--gen`` tokens each, one at a
time, and reports decode tok/s (the headline ``value``), prefill tok/s, time to first token and speculation acceptance.  Times are
host wall-clock around whole requests - what a client of the server sees minus HTTP - with a device synchronise at both ends of a
request on GPU engines.  The report has the shape ``autoconfig/compare.py`` reads, so a derived configuration can be compared with a
hand-written one.

    python -m layerstorm_b200.autoconfig.benchmark --prompt-len 8192 --gen 128 --requests 3 -- --autoconfig --model glm-5.3-flash --random-weights

Reference counterpart: python/autoconfig/benchmark.py (AUTO_RUN benchmark mode: measure a derived recipe, then exit).
"""
from __future__ import annotations

import argparse
import json
import statistics
import sys
import time
from typing import List, Optional


def measure(orch, vocab: int, prompt_len: int, gen: int, requests: int, warmup_len: int = 64, sync=None) -> dict:
    from ..serving.orchestrator import InferenceRequest, SamplingParams
    sync = sync or (lambda: None)

    def run(tag: str, n: int, salt: int):
        prompt = [(salt * 7919 + 13 * i) % max(vocab - 8, 1) + 4 for i in range(n)]         # distinct per request: no prefix-cache hits
        req = InferenceRequest(tag, prompt, SamplingParams(max_tokens=gen, temperature=0.0, ignore_eos=True))
        sync()
        t0 = time.perf_counter()
        orch.submit_request(req)
        while not req.done.is_set():
            if not orch.step():
                break
        sync()
        wall = time.perf_counter() - t0
        if req.error is not None:
            raise RuntimeError(f"{tag}: {req.error}")
        return req, wall

    run("warmup", warmup_len, 0)
    ttft, dec, pre, walls, rounds, accepted = [], [], [], [], 0, 0
    for i in range(requests):
        req, wall = run(f"bench{i}", prompt_len, i + 1)
        st = req.stats
        ttft.append(st.ttft_s * 1e3)
        dec.append(st.decode_tok_s)
        pre.append((st.prompt_tokens - st.cached_tokens) / st.ttft_s if st.ttft_s > 0 else 0.0)
        walls.append(wall)
        rounds += st.spec_rounds
        accepted += st.spec_accepted
    med = statistics.median
    return {"metric": "decode_tok_s", "value": round(med(dec), 3), "unit": "tok/s", "higher_is_better": True,
            "requests": requests, "prompt_len": prompt_len, "gen": gen,
            "extra": {"prefill_tok_s": round(med(pre), 1), "ttft_ms": round(med(ttft), 3), "request_wall_ms": round(med(walls) * 1e3, 3),
                      "spec_accepted_per_round": round(accepted / rounds, 3) if rounds else 0.0}}


def main(argv: Optional[List[str]] = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    serve_argv = argv[argv.index("--") + 1:] if "--" in argv else []
    own = argv[: argv.index("--")] if "--" in argv else argv
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--prompt-len", type=int, default=8192)
    ap.add_argument("--gen", type=int, default=128)
    ap.add_argument("--requests", type=int, default=3)
    ap.add_argument("--out", help="also write the report here")
    a = ap.parse_args(own)
    from ..cli import serve
    sargs = serve.build_parser().parse_args(serve_argv)
    cfg, shape, ckpt, _ = serve.resolve_config(sargs)
    need = a.prompt_len + a.gen + 8
    if cfg["serving"]["max_sequence_length"] < need:
        print(f"serving.max_sequence_length {cfg['serving']['max_sequence_length']} < prompt + generation ({need})", file=sys.stderr)
        return 2
    engine = serve.build_engine(cfg, shape, ckpt, sargs)
    _, orch = serve.build_server(cfg, shape, ckpt, engine, sargs)
    sync = None
    if not sargs.test_engine:
        import torch
        sync = torch.cuda.synchronize
    rep = measure(orch, getattr(engine, "vocab", None) or shape.vocab, a.prompt_len, a.gen, a.requests, sync=sync)
    rep["config"] = {"model": shape.name, "tp": cfg["parallelism"]["tensor_parallelism"], "kv": cfg["quantization"]["kv_cache"],
                     "prefill_chunk": cfg["orchestrator"]["prefill_chunk_tokens"], "speculation": cfg["speculation"]["method"]}
    line = json.dumps(rep)
    if a.out:
        with open(a.out, "w") as fh:
            fh.write(line + "\n")
    print(line)
    return 0


if __name__ == "__main__":
    sys.exit(main())
