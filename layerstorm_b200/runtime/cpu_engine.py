"""CPU engine: the engine interface (sequences, prefill, decode, verify rows, rewind, fork) on the host, for the
"CPU plumbing" configuration and as an end-to-end oracle.  Attention / norms / routing run through the fp32
reference model; the routed and shared experts run either there or - with ``native_experts=True`` - through the
native CPU expert kernels on slot images in any of the device formats (BF16, FP8 block, NVFP4, GGUF Q4_K), i.e. on
the same bytes the GPU kernels read.  Every step recomputes the whole sequence (O(T^2)); this is a correctness and
plumbing vehicle for tiny models, not a serving path.
Reference role: null / CPU backends of the daemon and the CPU expert device
(src/compute/cpu/numa_cpu_expert_device.*, BASELINE "CPU plumbing" configuration).
"""
from __future__ import annotations

import ctypes
import time
from typing import Dict, List, Optional, Sequence

import torch

from ..models.config import ModelConfig
from ..models.reference import Oracle, route, route_hash
from . import native as rt


class _ExpertOracle(Oracle):
    """Reference model whose MoE layers call the native CPU expert kernels."""

    def __init__(self, cfg: ModelConfig, weights, expert_quant: str, threads: int = 0):
        super().__init__(cfg, weights)
        from ..models.device_model import ExpertArena, QLinear, expert_layout
        self.cpu = rt.CpuExperts(threads)
        self.ef = expert_layout(expert_quant, cfg.hidden, cfg.moe_inter)
        self.arenas: Dict[int, "ExpertArena"] = {}
        E = cfg.n_routed + cfg.n_shared
        for i in range(cfg.n_layers):
            if not cfg.is_moe_layer(i):
                continue
            ar = ExpertArena(self.ef, E, E, "cpu")
            m = f"layers.{i}.moe."
            for e in range(E):
                nm = m + (f"experts.{e}." if e < cfg.n_routed else f"shared.{e - cfg.n_routed}.")
                ar.write_expert(e, *(QLinear.from_float(self.w[nm + t], expert_quant, "cpu") for t in ("gate", "up", "down")))
            self.arenas[i] = ar

    def ffn(self, i, x):
        cfg = self.cfg
        if not cfg.is_moe_layer(i):
            return super().ffn(i, x)
        m = f"layers.{i}.moe."
        logits = x @ self.w[m + "router"].T
        if cfg.is_hash_layer(i) and (m + "tid2eid") in self.tables:
            # hash layer: experts from the token-id table; a dropped slot (-1) becomes expert 0 with weight 0 for the native kernel
            ids, wt = route_hash(cfg, logits, self.tables[m + "tid2eid"], self._tok)
            wt = torch.where(ids >= 0, wt, torch.zeros(()))
            ids = ids.clamp_min(0)
        else:
            ids, wt = route(cfg, logits, self.w.get(m + "router_bias"))
        T = x.shape[0]
        if cfg.n_shared:
            sh = torch.arange(cfg.n_routed, cfg.n_routed + cfg.n_shared).expand(T, -1)
            ids = torch.cat([ids, sh], 1)
            wt = torch.cat([wt, torch.ones(T, cfg.n_shared)], 1)
        ar = self.arenas[i]
        slots = {e: ar.data[e] for e in range(cfg.n_routed + cfg.n_shared)}
        return self.cpu.moe_layer(ctypes.addressof(self.ef), slots, cfg.n_routed + cfg.n_shared, x, ids.int(), wt, cfg.swiglu_limit)


class CpuEngine:
    has_recurrent_state = False

    def __init__(self, cfg: ModelConfig, weights, native_experts: bool = True, expert_quant: str = "bf16", max_seqs: int = 8,
                 max_ctx: int = 4096, threads: int = 0):
        self.cfg, self.vocab, self.max_ctx, self.max_seqs = cfg, cfg.vocab, max_ctx, max_seqs
        self.model = _ExpertOracle(cfg, weights, expert_quant, threads) if native_experts else Oracle(cfg, weights)
        self.seqs: Dict[int, List[int]] = {}
        self._next = 0
        self.forward_seconds = 0.0

    def reduced_expert_view(self, top_k: int) -> "CpuEngine":
        """A second engine over the SAME weights that routes to ``top_k`` experts per token instead of the model's (own sequences):
        the draft side of self-speculative decoding."""
        import copy
        import dataclasses
        view = copy.copy(self)
        view.cfg = dataclasses.replace(self.cfg, top_k=max(1, min(top_k, self.cfg.top_k)))
        view.model = copy.copy(self.model)
        view.model.cfg = view.cfg
        view.model.sel_log = {}
        view.seqs, view._next, view.forward_seconds = {}, 0, 0.0
        return view

    # ---- sequences ----
    def create_sequence(self) -> int:
        if len(self.seqs) >= self.max_seqs:
            raise RuntimeError("no free sequence slot")
        self._next += 1
        self.seqs[self._next] = []
        return self._next

    def free_sequence(self, sid: int):
        self.seqs.pop(sid)

    def fork_sequence(self, parent: int, prefix_len: Optional[int] = None) -> int:
        sid = self.create_sequence()
        src = self.seqs[parent]
        self.seqs[sid] = list(src if prefix_len is None else src[:prefix_len])
        return sid

    def rewind(self, sid: int, length: int):
        del self.seqs[sid][length:]

    def seq_len(self, sid: int) -> int:
        return len(self.seqs[sid])

    def free_page_count(self) -> int:
        return 1 << 30

    # ---- compute ----
    def _logits(self, toks: Sequence[int]) -> torch.Tensor:
        if len(toks) > self.max_ctx:
            raise RuntimeError("context length exceeded")
        t0 = time.perf_counter()
        out = self.model.forward(torch.tensor(list(toks)))
        self.forward_seconds += time.perf_counter() - t0
        return out

    def prefill(self, sid: int, tokens: Sequence[int], want_logits: bool = False):
        s = self.seqs[sid]
        s.extend(int(t) for t in tokens)
        lg = self._logits(s)[-1]
        nxt = int(torch.argmax(lg))
        return (nxt, lg) if want_logits else nxt

    def decode(self, sids: Sequence[int], tokens: Sequence[int], return_logits: bool = False):
        outs, lgs = [], []
        for sid, t in zip(sids, tokens):
            self.seqs[sid].append(int(t))
            lg = self._logits(self.seqs[sid])[-1]
            outs.append(int(torch.argmax(lg)))
            lgs.append(lg)
        return (outs, torch.stack(lgs)) if return_logits else outs

    def forward_rows(self, sid: int, tokens: Sequence[int], commit: bool = True) -> torch.Tensor:
        s = self.seqs[sid]
        n0 = len(s)
        lg = self._logits(s + [int(t) for t in tokens])[n0:]
        if commit:
            s.extend(int(t) for t in tokens)
        return lg


def cpu_plumbing_run(native_experts: bool = True, expert_quant: str = "bf16", prompt_len: int = 64, new_tokens: int = 32, seed: int = 0):
    """The CPU configuration of the benchmark suite: tiny MLA-MoE decoder (4 layers, hidden 256, 16 experts top-4 + 1 shared),
    fp32 N(0, 0.02) weights, a uniform-random prompt, greedy decode.  Returns (tokens, seconds, tok/s)."""
    from ..models.config import get_preset
    from ..models.weights import init_weights
    cfg = get_preset("tiny-mla-moe")
    w = init_weights(cfg, seed)
    eng = CpuEngine(cfg, w, native_experts=native_experts, expert_quant=expert_quant)
    g = torch.Generator().manual_seed(seed)
    prompt = torch.randint(0, cfg.vocab, (prompt_len,), generator=g).tolist()
    sid = eng.create_sequence()
    t0 = time.perf_counter()
    tok = eng.prefill(sid, prompt)
    out = [tok]
    for _ in range(new_tokens - 1):
        tok = eng.decode([sid], [tok])[0]
        out.append(tok)
    dt = time.perf_counter() - t0
    return out, dt, new_tokens / dt
