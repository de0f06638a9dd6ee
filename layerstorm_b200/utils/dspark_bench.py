"""Time the block draft: context ingest per chunk and one block pass, per weight format.

    python -m layerstorm_b200.utils.dspark_bench [--geometry shipped|small] [--formats bf16,fp8_e4m3,nvfp4] [--context 8192] [--chunk 2048]
                                                 [--rows 8] [--iters 20] [--device cuda]

``shipped`` is the geometry of the published GLM-5.2 dspark speculator (5 dense layers of width 6144, 64 heads of 64, MLP 12288,
154880-token vocabulary, 5 aux layers: 7.6 GB in bf16); ``small`` a 2-layer draft of width 1024 for a quick look.  Random weights,
made on the device.  Per format one JSON line: bytes of the draft's weights, ms per ingested chunk (and rows/s), ms per block pass of
``--rows`` rows over a context of ``--context`` positions, and the weight sweep that pass implies in GB/s (weights read once per pass:
the figure to hold against the measured copy bandwidth of the GPU).  On the GPU the time is taken with CUDA events after warm-up;
on the CPU (``--device cpu``, library GEMMs in fp32, formats ignored) with the wall clock - useful only for the small geometry.
Reference: the draft step timing of src/speculation/dspark_runtime.cpp (LS_DSPARK_PROF).
"""
from __future__ import annotations

import argparse
import json
import sys
import time
from typing import Optional, Sequence

import torch

from ..speculation import dspark as dsp


def geometry(name: str) -> dsp.DsparkCheckpointConfig:
    if name == "shipped":
        c = dsp.DsparkCheckpointConfig(draft_vocab_size=154880, mask_token_id=154856, aux_hidden_state_layer_ids=[8, 23, 39, 55, 70], hidden_size=6144,
                                       num_attention_heads=64, num_key_value_heads=64, head_dim=64, intermediate_size=12288, vocab_size=154880,
                                       enable_confidence_head=True, confidence_head_with_markov=True)
    elif name == "small":
        c = dsp.DsparkCheckpointConfig(num_hidden_layers=2, markov_rank=64, draft_vocab_size=32768, mask_token_id=32767, aux_hidden_state_layer_ids=[2, 5, 8],
                                       hidden_size=1024, num_attention_heads=16, num_key_value_heads=16, head_dim=64, intermediate_size=2048, vocab_size=32768,
                                       enable_confidence_head=True, confidence_head_with_markov=True)
    else:
        raise ValueError(f"unknown geometry {name!r}")
    c.check()
    return c


def _timed(fn, iters: int, cuda: bool) -> float:
    """Milliseconds per call (median of ``iters`` after three warm-up calls)."""
    for _ in range(3):
        fn()
    times = []
    if cuda:
        torch.cuda.synchronize()
        for _ in range(iters):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            b.synchronize()
            times.append(a.elapsed_time(b))
    else:
        for _ in range(iters):
            t0 = time.perf_counter()
            fn()
            times.append((time.perf_counter() - t0) * 1e3)
    times.sort()
    return times[len(times) // 2]


def run(cfg: dsp.DsparkCheckpointConfig, fmt: Optional[str], device: str, context: int, chunk: int, rows: int, iters: int, seed: int = 0) -> dict:
    cuda = torch.device(device).type == "cuda"
    tens = dsp.random_dspark_tensors(cfg, seed, torch.bfloat16 if cuda else torch.float32, device)
    bb = dsp.DsparkBackbone(cfg, tens, device, None if cuda else torch.float32, ctx_capacity=max(context + chunk, 4 * cfg.block_size), rotate=False,
                            kernels=fmt if cuda else None)
    del tens
    ctx = bb.new_context()
    g = torch.Generator(device=device).manual_seed(seed + 1)
    aux = torch.randn(chunk, cfg.n_aux * cfg.hidden_size, generator=g, device=device, dtype=bb.dtype)
    pos = 0
    while pos < context:                                        # fill the context chunk by chunk
        n = min(chunk, context - pos)
        bb.ingest(ctx, aux[:n], pos)
        pos += n

    def ingest():
        ctx.length = context                                    # the same chunk again, at the end of the filled context
        bb.ingest(ctx, aux, context)
    ms_ingest = _timed(ingest, max(3, iters // 4), cuda)
    ctx.length = context
    ms_block = _timed(lambda: bb.run_block(ctx, 5, context, rows - 1), iters, cuda)
    ms_draft = _timed(lambda: bb.draft(ctx, 5, context, rows - 1), max(3, iters // 4), cuda)
    wb = bb.weight_bytes() - bb.embed.numel() * bb.embed.element_size()          # a pass reads rows of the embedding, not the table
    return {"format": fmt if cuda else "fp32-cpu", "weight_bytes": bb.weight_bytes(), "context": context, "chunk_rows": chunk, "ingest_ms": round(ms_ingest, 3),
            "ingest_rows_per_s": round(chunk / ms_ingest * 1e3), "block_rows": rows, "block_ms": round(ms_block, 3), "draft_ms_with_heads": round(ms_draft, 3),
            "weight_sweep_gb_s": round(wb / ms_block / 1e6, 1), "context_bytes": ctx.k.numel() * ctx.k.element_size() * 2}


def main(argv: Optional[Sequence[str]] = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--geometry", default="shipped")
    ap.add_argument("--formats", default="bf16,fp8_e4m3,nvfp4")
    ap.add_argument("--context", type=int, default=8192)
    ap.add_argument("--chunk", type=int, default=2048)
    ap.add_argument("--rows", type=int, default=8)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--device", default="cuda")
    a = ap.parse_args(argv)
    try:
        cfg = geometry(a.geometry)
    except ValueError as e:
        print(str(e), file=sys.stderr)
        return 2
    if a.rows < 2 or a.rows > cfg.block_size:
        print(f"--rows must be 2 .. {cfg.block_size} (the anchor row + predicting rows)", file=sys.stderr)
        return 2
    fmts = [f for f in a.formats.split(",") if f] if torch.device(a.device).type == "cuda" else [None]
    for fmt in fmts:
        print(json.dumps(dict(run(cfg, fmt, a.device, a.context, a.chunk, a.rows, a.iters), geometry=a.geometry)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
