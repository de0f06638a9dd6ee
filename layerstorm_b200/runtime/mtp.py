"""Multi-token-prediction (MTP) block 0 on the device, kept in step with the main model's sequences.

The block has a latent cache of its own over the sequence's pages (``DeviceModel.kv_cache[n_layers]``).  Its row for position p needs
the main model's stream at p (in front of the output norm) and the token at p + 1, so it always lags the main model by one position:
after the main model has consumed tokens t_0 .. t_{n-1} the block's cache is complete for positions 0 .. n-2, and position n-1 is run
as soon as t_n is known - which is also the row whose logits propose t_{n+1}, the draft token.

``MtpRunner`` keeps, per sequence, how many positions of the block's cache are valid and a small stash of the main model's streams of
the last step's rows (the rows a verify step accepted or not are all there; only the committed ones are ever consumed):
  * after every chunk of a prefill the block runs over the chunk's rows (token ahead = the next prompt token), except the last row of
    the last chunk, whose stream goes to the stash;
  * before any later step of the sequence, and in :meth:`draft`, the positions between the valid frontier and the committed frontier
    are run from the stash (``catch_up``);
  * a fork copies the parent's frontier and stash; a rewind pulls the frontier back to the last position whose token ahead survived.
A sequence whose stash no longer covers the missing positions (a fork below the parent's frontier, more rows in one step than the
stash holds) is marked out of step and proposes nothing from then on; speculation stays lossless either way, the target verifies.
One block (depth 1): a deeper draft needs one more lagging cache per depth and is left to the CPU reference (``models/mtp.py``).
Reference: the engine's MtpSpeculationMethod (src/speculation/) and python/orchestrator/mtp_draft.py.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch

from ..ops import _native as nat


class MtpRunner:
    STASH_ROWS = 16

    def __init__(self, engine):
        m = engine.model
        if not m.mtp_layers:
            raise NotImplementedError("the model has no multi-token-prediction block on the device (n_mtp = 0, hyper-connections, "
                                      "tensor parallelism or a 4-bit KV cache)")
        if engine.row_tier is not None or m.streamer is not None or getattr(m, "dcp", None) is not None:
            raise NotImplementedError("the device MTP block needs resident experts and an untiered, unsharded KV cache")
        self.eng = engine
        self.H = engine.cfg.hidden
        self.stash = torch.zeros(engine.max_seqs, self.STASH_ROWS, self.H, dtype=torch.float32, device=engine.dev)
        # sid -> [valid positions of the block's cache, first position in the stash, rows in the stash]; absent = out of step
        self.state: Dict[int, List[int]] = {sid: [0, 0, 0] for sid, s in engine.seqs.items() if s.length == 0}
        self._pins: List[torch.Tensor] = []
        self.block_rows = 0          # rows the block has run (statistics)
        self.last_ws = None          # workspace of the last catch-up (its logits row 0 = the last proposal's distribution)
        self.drafts = 0

    # ------------------------------------------------------------------ bookkeeping hooks
    def on_create(self, sid: int):
        self.state[sid] = [0, 0, 0]

    def on_free(self, sid: int):
        self.state.pop(sid, None)

    def on_fork(self, parent: int, child: int, prefix_len: int):
        st = self.state.get(parent)
        if st is None or st[0] < prefix_len - 1:
            self.state.pop(child, None)
            return
        self.stash[child].copy_(self.stash[parent])
        self.state[child] = [max(0, min(st[0], prefix_len - 1)), st[1], st[2]]

    def on_rewind(self, sid: int, length: int):
        st = self.state.get(sid)
        if st is not None:
            st[0] = max(0, min(st[0], length - 1))     # position length-1 was run with a token ahead that is gone

    def _resid(self, ws):
        return ws.resid.view(-1)[: ws.R * self.H].view(ws.R, self.H)

    def stash_rows(self, sid: int, ws, row0: int, n: int, base_pos: int):
        """Keep the main model's streams of rows [row0, row0 + n) of the step just run (positions base_pos ..)."""
        if sid not in self.state:
            return
        if n > self.STASH_ROWS:
            row0, base_pos, n = row0 + n - self.STASH_ROWS, base_pos + n - self.STASH_ROWS, self.STASH_ROWS
        self.stash[sid, :n].copy_(self._resid(ws)[row0: row0 + n])
        st = self.state[sid]
        st[1], st[2] = base_pos, n

    # ------------------------------------------------------------------ the block
    def catch_up(self, sid: int, next_tok: int, want_draft: bool = False) -> Optional[int]:
        """Run the block over the positions between its valid frontier and the sequence's committed frontier; ``next_tok`` is the
        token that follows the last committed one.  With ``want_draft`` returns the block's arg-max at the last position (its
        proposal for the token after ``next_tok``), else None.  Must be called before the main step that consumes ``next_tok``
        is staged."""
        eng = self.eng
        st = self.state.get(sid)
        s = eng.seqs[sid]
        if st is None or s.length == 0:
            return None
        lo, hi = st[0], s.length - 1
        if lo > hi:
            if not want_draft:
                return None
            lo = hi                                     # in step already: the last position again, for its logits
        base, n = st[1], st[2]
        if lo < base or hi >= base + n or hi - lo + 1 > self.STASH_ROWS:
            self.state.pop(sid, None)                   # the streams of the missing positions are gone
            return None
        rows = [((int(s.tokens[p + 1]) if p + 1 < s.length else int(next_tok)), s.slot, p) for p in range(lo, hi + 1)]
        R = len(rows)
        ws = eng._ws_rows(R)
        self.last_ws = ws
        out = None
        with torch.cuda.stream(eng.stream):
            eng._stage(ws, rows, [(0, R, s.slot)])
            self._resid(ws)[:R].copy_(self.stash[sid, lo - base: hi - base + 1])
            n0 = nat.launch_count()
            eng.model.forward_mtp(ws, R, 0, R - 1, 1 if want_draft else 0)
            if want_draft:
                eng.model.argmax(ws, 1)
                eng.h_out[:1].copy_(ws.out_tok[:1], non_blocking=True)
                eng.d2h_bytes += 4
                eng._queue_error_readback()
                eng.stream.synchronize()
                eng._check_errors()
                out = int(eng.h_out[0])
            eng.kernel_launches += nat.launch_count() - n0
        st[0] = hi + 1
        self.block_rows += R
        return out

    def before_step(self, sid: int, first_tok: int):
        st = self.state.get(sid)
        if st is not None and st[0] < self.eng.seqs[sid].length:
            self.catch_up(sid, first_tok, want_draft=False)

    def after_prefill_chunk(self, sid: int, ws, chunk: Sequence[int], pos0: int, next_tok: Optional[int]):
        """The block over the rows of a prefill chunk the main model has just run (workspace ``ws``, rows at positions pos0 ..);
        ``next_tok``: the prompt token after the chunk, None for the last chunk (its last row waits in the stash)."""
        st = self.state.get(sid)
        if st is None:
            return
        if st[0] != pos0:
            self.state.pop(sid, None)
            return
        eng = self.eng
        R = len(chunk)
        Rm = R if next_tok is not None else R - 1
        if next_tok is None:
            self.stash[sid, 0].copy_(self._resid(ws)[R - 1])
            st[1], st[2] = pos0 + R - 1, 1
        else:
            st[2] = 0
        if Rm > 0:
            ahead = torch.tensor(list(chunk[1:]) + ([int(next_tok)] if next_tok is not None else []), dtype=torch.int32).pin_memory()
            self._pins.append(ahead)                    # alive until the prefill's synchronize
            ws.tok[:Rm].copy_(ahead, non_blocking=True)
            eng.h2d_bytes += 4 * Rm
            eng.model.forward_mtp(ws, Rm, 0, 0, 0)
            self.block_rows += Rm
        st[0] = pos0 + Rm

    def release_pins(self):
        self._pins.clear()

    def draft(self, sid: int, next_tok: int) -> List[int]:
        """The block's proposal for the token after ``next_tok`` (one token, or nothing when the sequence is out of step)."""
        t = self.catch_up(sid, next_tok, want_draft=True)
        if t is None:
            return []
        self.drafts += 1
        return [t]
