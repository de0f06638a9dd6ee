"""Expert slot images built straight from a GGUF file, for the pinned host store of a capped expert cache.

``ExpertStreamer.add_layer`` normally receives a layer whose experts were first assembled in a full device arena and copies them
to pinned host memory.  For a GGUF checkpoint whose expert tensors are stored in block types the kernels read natively (Q4_K, Q5_K,
Q6_K, Q8_0) that detour is unnecessary: a slot image is the expert's gate | up | down blocks in their device layouts (Q4_K / Q5_K
verbatim, Q6_K padded to 224-byte blocks, Q8_0 split into a quant plane and a scale plane) followed by zeros up to the slot stride.
``LiveGgufExpertSource`` produces exactly those bytes from the memory-mapped file, per (layer, expert), from any thread (NumPy
copies release the interpreter lock); ``build_layer`` fills a layer's host slots with a small thread pool.  The result is
byte-identical to the slot the device path writes (``ExpertArena.write_expert`` of ``QLinear.from_ggml`` matrices), which the
tests check.  Layers with a tensor in another type, or with gate and up in different types, are not covered (``layout`` returns
None) and go the ordinary way.
Reference: src/model/weight_pipeline/live_gguf_source.h:1-70 (live prepack: slot bytes from the source GGUF, byte-identical to the
offline prepack, no CUDA), live_arena_build.h (worker pool committing straight into the pinned arena).
"""
from __future__ import annotations

from concurrent.futures import ThreadPoolExecutor
from typing import Dict, Optional, Sequence

import numpy as np
import torch


class LiveGgufExpertSource:
    def __init__(self, ckpt, cfg, expert_width: Optional[int] = None, threads: int = 8):
        """``ckpt``: a ``LazyCheckpoint`` over a GGUF file (``native_ggml``); ``cfg``: the model shape."""
        if not hasattr(ckpt, "native_ggml") or getattr(ckpt, "kind", "gguf") != "gguf":
            raise ValueError("a live expert source needs a GGUF checkpoint (file-order blocks through native_ggml)")
        self.ck, self.cfg, self.threads = ckpt, cfg, max(1, threads)
        self.F = expert_width or cfg.moe_inter
        self._layouts: Dict[int, object] = {}
        self.bytes_built = 0

    def _name(self, layer: int, e: int) -> str:
        c = self.cfg
        return f"layers.{layer}.moe." + (f"experts.{e}." if e < c.n_routed else f"shared.{e - c.n_routed}.")

    def layout(self, layer: int):
        """The slot layout (``ExpertFmt``) of the layer when every expert's three matrices are natively readable with one type for
        gate / up and one for down, else None."""
        if layer in self._layouts:
            return self._layouts[layer]
        from ..formats import gguf as g
        from ..models.device_model import expert_layout
        c, ef = self.cfg, None
        if c.is_moe_layer(layer) and c.hidden % 256 == 0 and self.F % 256 == 0 and self.F == c.moe_inter:
            types = set()
            for e in range(c.n_routed + c.n_shared):
                t = [self.ck.native_ggml(self._name(layer, e) + p) for p in ("gate", "up", "down")]
                if any(x is None for x in t):
                    types = None
                    break
                types.add((t[0][0], t[1][0], t[2][0]))
            if types and len(types) == 1:
                tg, tu, td = next(iter(types))
                if tg == tu and tg in g.DEVICE_NATIVE and td in g.DEVICE_NATIVE:
                    ef = expert_layout(g.DEVICE_NATIVE[tg], c.hidden, self.F, g.DEVICE_NATIVE[td])
        self._layouts[layer] = ef
        return ef

    def load_into(self, layer: int, expert: int, dst: np.ndarray):
        """Write the slot image of one expert into ``dst`` (uint8, at least the slot stride long)."""
        from ..formats import gguf as g
        ef = self.layout(layer)
        if ef is None:
            raise ValueError(f"layer {layer} is not covered by the live source")
        dst[: ef.stride] = 0
        nm = self._name(layer, expert)
        for proj, off in (("gate", ef.off_gate), ("up", ef.off_up), ("down", ef.off_down)):
            t, raw, rows, cols = self.ck.native_ggml(nm + proj)
            d = g.to_device_layout(t, raw, rows, cols).reshape(-1)
            dst[off: off + d.size] = d
        self.bytes_built += int(ef.stride)

    def build_layer(self, layer: int, experts: Sequence[int], host: torch.Tensor, rows: Optional[Sequence[int]] = None):
        """Fill ``host[rows[j]]`` (pinned uint8 [n, stride]) with the slot image of ``experts[j]``, ``threads`` at a time."""
        arr = host.numpy()
        rows = list(rows) if rows is not None else list(range(len(experts)))
        with ThreadPoolExecutor(max_workers=self.threads) as pool:
            list(pool.map(lambda je: self.load_into(layer, je[1], arr[je[0]]), zip(rows, experts)))
