"""CPU stand-in for the GPU step engine with the same public surface.

It plays the role of the reference's null backends (``EngineBackends null_backends()``,
src/daemon/engine.h:98-108, pybind ``start_engine_test``): the whole control plane -
orchestrator, prefix cache, speculation loops, HTTP server - runs and is tested without CUDA.
The "model" is a deterministic hash of the token prefix, so outputs are reproducible and
depend on the full context (a wrong KV rewind or a wrong fork shows up as different tokens).
"""
from __future__ import annotations

import hashlib
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import torch

from .native import KvPoolExhausted, PageAllocator


@dataclass
class _Seq:
    slot: int
    tokens: List[int] = field(default_factory=list)

    @property
    def length(self) -> int:
        return len(self.tokens)


class NullEngine:
    """Deterministic fake model.  ``vocab`` tokens; logits are a hash-seeded pseudo-random vector
    with one strongly preferred token, optionally scripted through ``script`` (a dict mapping a
    prefix tuple to the next token)."""

    def __init__(self, vocab: int = 512, max_seqs: int = 8, max_ctx: int = 4096, page: int = 16, num_pages: Optional[int] = None,
                 eos_token: int = 1, script: Optional[Dict[tuple, int]] = None, has_recurrent_state: bool = False):
        self.vocab, self.max_seqs, self.max_ctx, self.page = vocab, max_seqs, max_ctx, page
        self.num_pages = num_pages if num_pages is not None else max_seqs * ((max_ctx + page - 1) // page)
        self.pa = PageAllocator([self.num_pages], page)
        self.free_slots = list(range(max_seqs - 1, -1, -1))
        self.seqs: Dict[int, _Seq] = {}
        self.eos_token = eos_token
        self.script = script or {}
        self.has_recurrent_state = has_recurrent_state
        self.kernel_launches = 0
        self.steps = 0
        self.prefill_tokens = 0

    # ---- model ----
    def _next(self, toks: Sequence[int]) -> int:
        key = tuple(toks)
        if key in self.script:
            return self.script[key]
        h = hashlib.blake2b(bytes(str(key[-64:]), "utf8") + len(key).to_bytes(4, "little"), digest_size=8).digest()
        return 2 + int.from_bytes(h, "little") % (self.vocab - 2)

    def _logits(self, toks: Sequence[int]) -> torch.Tensor:
        nxt = self._next(toks)
        g = torch.Generator().manual_seed(hash(tuple(toks[-8:])) & 0x7FFFFFFF)
        lg = torch.randn(self.vocab, generator=g)
        lg[nxt] = lg.max() + 4.0
        return lg

    # ---- sequences ----
    def create_sequence(self) -> int:
        if not self.free_slots:
            raise RuntimeError("no free sequence slot")
        s = self.free_slots.pop()
        self.seqs[s] = _Seq(s)
        self.pa.create(s)
        return s

    def free_sequence(self, sid: int):
        self.seqs.pop(sid)
        self.pa.destroy(sid)
        self.free_slots.append(sid)

    def fork_sequence(self, parent: int, prefix_len: Optional[int] = None) -> int:
        ps = self.seqs[parent]
        prefix_len = ps.length if prefix_len is None else prefix_len
        if self.has_recurrent_state and prefix_len != ps.length:
            raise RuntimeError("a sequence with recurrent state can only be forked at its frontier")
        if not self.free_slots:
            raise RuntimeError("no free sequence slot")
        s = self.free_slots.pop()
        self.pa.fork(parent, s, prefix_len)
        self.seqs[s] = _Seq(s, list(ps.tokens[:prefix_len]))
        return s

    def rewind(self, sid: int, length: int):
        s = self.seqs[sid]
        if self.has_recurrent_state and length < s.length:
            raise RuntimeError("rewind of a recurrent-state sequence is refused")
        del s.tokens[length:]
        self.pa.rewind(sid, length)

    def seq_len(self, sid: int) -> int:
        return self.seqs[sid].length

    def free_page_count(self) -> int:
        return self.pa.free_pages(0)

    def _grow(self, sid: int, n: int):
        s = self.seqs[sid]
        if s.length + n > self.max_ctx:
            raise RuntimeError(f"sequence length {s.length + n} exceeds max context {self.max_ctx}")
        self.pa.cow_frontier(sid)
        self.pa.extend(sid, s.length + n)

    # ---- steps ----
    def prefill(self, sid: int, tokens: Sequence[int], want_logits: bool = False):
        self._grow(sid, len(tokens))
        s = self.seqs[sid]
        s.tokens.extend(int(t) for t in tokens)
        self.prefill_tokens += len(tokens)
        self.steps += 1
        lg = self._logits(s.tokens)
        nxt = int(lg.argmax())
        return (nxt, lg) if want_logits else nxt

    def decode(self, sids: Sequence[int], tokens: Sequence[int], return_logits: bool = False):
        outs, lgs = [], []
        for sid in sids:
            self._grow(sid, 1)                # every sequence gets its page before any advances: a step that runs out of pages can be run again
        for sid, t in zip(sids, tokens):
            s = self.seqs[sid]
            s.tokens.append(int(t))
            lg = self._logits(s.tokens)
            outs.append(int(lg.argmax()))
            lgs.append(lg)
        self.steps += 1
        return (outs, torch.stack(lgs)) if return_logits else outs

    def forward_rows(self, sid: int, tokens: Sequence[int], commit: bool = True) -> torch.Tensor:
        """Logits for every row of a run of consecutive tokens (speculative verify shape)."""
        self._grow(sid, len(tokens))
        s = self.seqs[sid]
        base = list(s.tokens)
        rows = []
        for t in tokens:
            base.append(int(t))
            rows.append(self._logits(base))
        if commit:
            s.tokens = base
        else:
            self.pa.rewind(sid, s.length)
        self.steps += 1
        return torch.stack(rows)
