"""Run-to-run determinism probe and drift diff.

``probe``  sends one warm-up request, then the same greedy request ``reps`` times through an ``Orchestrator`` (prefix cache bypassed by
           a unique leading token per warm-up only - the probe requests themselves are identical, so with the prefix cache enabled the
           later ones also exercise the fork path) and reports every run's tokens, the pairwise first divergence and a verdict.
           Exit code of the CLI: 0 = all runs identical, 1 = divergence.
``drift``  compares two dumps of per-layer activations (``.npz`` files written by any two runs: same keys, same shapes) and reports, per
           key, max abs / relative error and the first key whose relative error exceeds a tolerance - the place where two runs (eager vs
           CUDA graph, 1 GPU vs N GPUs, two builds) start to differ.

    python -m layerstorm_b200.utils.determinism_probe probe --model tiny-mla-moe --prompt-len 512 --gen 16 --reps 3
    python -m layerstorm_b200.utils.determinism_probe probe --model glm-5.3-flash --layers 8 --prompt-len 4096 --gen 8   # full-width slice
    python -m layerstorm_b200.utils.determinism_probe drift a.npz b.npz --rtol 1e-3

Reference counterparts: tools/serve_determinism_probe.py (warm-up, identical greedy repetitions, pairwise first divergence, verdict) and
tools/drift_dump_diff.py.
"""
from __future__ import annotations

import argparse
import json
import sys
from typing import Dict, List, Optional, Sequence


def first_divergence(a: Sequence[int], b: Sequence[int]) -> int:
    """Index of the first differing token; -1 when identical."""
    for i, (x, y) in enumerate(zip(a, b)):
        if x != y:
            return i
    return -1 if len(a) == len(b) else min(len(a), len(b))


def probe(orch, prompt: Sequence[int], gen: int = 16, reps: int = 3, warmup_prompt: Optional[Sequence[int]] = None, step=None) -> dict:
    """``step``: callable that drives the orchestrator until a request is done (default: ``orch.step()`` in this thread)."""
    from ..serving.orchestrator import InferenceRequest, SamplingParams

    def run(tag, toks):
        req = InferenceRequest(tag, list(toks), SamplingParams(max_tokens=gen, temperature=0.0, ignore_eos=True))
        orch.submit_request(req)
        if step is None:
            while not req.done.is_set():
                if not orch.step():
                    break
        else:
            step(req)
        if req.error is not None:
            raise RuntimeError(f"{tag}: {req.error}")
        return list(req.output_ids)

    if warmup_prompt:
        run("warmup", warmup_prompt)
    runs = [run(f"probe{i}", prompt) for i in range(reps)]
    pairs = {f"{i}-{j}": first_divergence(runs[i], runs[j]) for i in range(reps) for j in range(i + 1, reps)}
    return {"reps": reps, "prompt_tokens": len(prompt), "generated": gen, "runs": runs, "first_divergence": pairs,
            "identical": all(v < 0 for v in pairs.values())}


def drift(a: Dict[str, "object"], b: Dict[str, "object"], rtol: float = 1e-3) -> dict:
    import numpy as np
    rows, first = [], None
    for k in a:
        if k not in b:
            rows.append({"key": k, "missing_in_b": True})
            continue
        x, y = np.asarray(a[k], np.float64), np.asarray(b[k], np.float64)
        if x.shape != y.shape:
            rows.append({"key": k, "shape_a": list(x.shape), "shape_b": list(y.shape)})
            first = first or k
            continue
        err = float(np.abs(x - y).max()) if x.size else 0.0
        rel = err / (float(np.abs(x).max()) + 1e-30)
        rows.append({"key": k, "max_abs": err, "rel": rel})
        if first is None and rel > rtol:
            first = k
    return {"keys": len(rows), "first_over_tolerance": first, "rtol": rtol, "rows": rows, "only_in_b": [k for k in b if k not in a]}


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    sub = ap.add_subparsers(dest="cmd", required=True)
    p = sub.add_parser("probe")
    p.add_argument("--model", default="tiny-mla-moe")
    p.add_argument("--test-engine", action="store_true", help="CPU null engine instead of a GPU model")
    p.add_argument("--prompt-len", type=int, default=512)
    p.add_argument("--gen", type=int, default=16)
    p.add_argument("--reps", type=int, default=3)
    p.add_argument("--warmup-len", type=int, default=64)
    p.add_argument("--prefix-cache", action="store_true")
    p.add_argument("--layers", type=int, default=0, help="keep the first N layers of the model shape at full width (a slice of a large model)")
    p.add_argument("--prefill-chunk", type=int, default=2048)
    d = sub.add_parser("drift")
    d.add_argument("a")
    d.add_argument("b")
    d.add_argument("--rtol", type=float, default=1e-3)
    a = ap.parse_args(argv)
    if a.cmd == "drift":
        import numpy as np
        rep = drift(dict(np.load(a.a)), dict(np.load(a.b)), a.rtol)
        print(json.dumps({k: v for k, v in rep.items() if k != "rows"}))
        for r in rep["rows"]:
            print(json.dumps(r))
        return 0 if rep["first_over_tolerance"] is None else 1
    from ..serving.orchestrator import Orchestrator
    from ..serving.prefix_cache import PrefixCacheConfig
    if a.test_engine:
        from ..runtime.null_engine import NullEngine
        eng = NullEngine()
        vocab = eng.vocab
    else:
        import torch
        from ..models.config import get_preset
        from ..models.device_model import DeviceModel
        from ..runtime.engine import Engine
        shape = get_preset(a.model)
        if a.layers and a.layers < shape.n_layers:
            import dataclasses
            shape = dataclasses.replace(shape, n_layers=a.layers, **({"layer_types": list(shape.layer_types[:a.layers])} if shape.layer_types else {}))
        dev = torch.device("cuda", 0)
        eng = Engine(DeviceModel.random_init(shape, dev, "fp8", 64, expert_slots="auto", embed_on_host=shape.vocab * shape.hidden > 2 ** 28,
                                             reserve_bytes=8 << 30),
                     max_seqs=8, max_ctx=a.prompt_len + a.gen + 64, prefill_chunk=a.prefill_chunk)
        vocab = shape.vocab
    orch = Orchestrator(eng, prefix_cache=PrefixCacheConfig(enabled=a.prefix_cache))
    prompt = [(7 + 13 * i) % (vocab - 8) + 4 for i in range(a.prompt_len)]
    warm = [(3 + 5 * i) % (vocab - 8) + 4 for i in range(a.warmup_len)]
    rep = probe(orch, prompt, a.gen, a.reps, warm)
    print(json.dumps(rep))
    return 0 if rep["identical"] else 1


if __name__ == "__main__":
    sys.exit(main())
