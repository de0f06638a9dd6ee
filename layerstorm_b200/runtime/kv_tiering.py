"""Row-granular KV tiering of ACTIVE sequences: old pages of a long sequence move to pinned host memory while the sequence keeps
decoding; the rows the sparse-attention indexer selects from them are fetched back row by row.

Only the latent KV cache is tiered.  The indexer's key cache (36 bytes per token and layer) stays in HBM with a page table of
its own, so every position can always be scored; what the scoring selects (at most ``index_topk`` rows per query row) is
materialised per attention layer in a dense buffer - rows of hot pages by ``lsb_kv_row_gather``, rows of cold pages through one
pinned host->device copy plus ``lsb_kv_row_scatter`` - and the ordinary attention kernel runs over that buffer.  Bytes move
verbatim, so tiered decoding equals untiered decoding bit for bit.

Bookkeeping: the native ``KvTierTable`` owns the cold slots (which logical page of which sequence sits where), the native
page allocator takes the HBM page back (``swap_out``) - the block-table entry of a cold page is -1.
Reference: KvTieringManager (src/daemon/kv_tiering_manager.h:66-127), kv_row_gather / kv_row_scatter
(src/compute/kernels/smxx/kv/kv_row_copy.cu:35,50).

Scope: decode-sized steps (and any step whose selected rows fit the staging buffer) of models whose attention layers all go
through the indexer's selection.  A prefill chunk that has to read cold rows is refused: prefill with the whole context hot,
then let the window slide.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from ..ops import _native as nat
from . import native as rt


class RowTiering:
    def __init__(self, engine, hot_window_tokens: int, cold_pages: int, max_staged_rows: int = 1 << 16):
        m = engine.model
        cfg = m.cfg
        if not cfg.has_indexer:
            raise ValueError("row-granular KV tiering needs sparse attention (an indexer): dense attention reads every row of every page")
        self.eng, self.model = engine, m
        self.page, self.rb = m.page, m.kv_row_bytes
        self.hot_window = max(hot_window_tokens, 2 * self.page)
        self.tier = rt.KvTierTable(self.page, self.hot_window, cold_pages, 0)
        self.cold_pages = cold_pages
        self.cold_kv: Dict[int, torch.Tensor] = {i: torch.empty(cold_pages, *t.shape[1:], dtype=t.dtype).pin_memory() for i, t in m.kv_cache.items()}
        self.cold_map: Dict[int, torch.Tensor] = {}          # sid -> int32 [max_pages]: cold slot of each logical page, -1 = hot
        self.next_page: Dict[int, int] = {}                  # sid -> first logical page not yet demoted
        self.copy_stream = torch.cuda.Stream(device=m.device)
        self.max_staged = max_staged_rows
        self.h_stage = torch.empty(max_staged_rows, self.rb, dtype=torch.uint8).pin_memory()
        self.h_dst = torch.empty(max_staged_rows, dtype=torch.int32).pin_memory()
        self.d_stage = torch.empty(max_staged_rows, self.rb, dtype=torch.uint8, device=m.device)
        self.d_dst = torch.empty(max_staged_rows, dtype=torch.int32, device=m.device)
        self.h_sel = None
        self._bufs: Dict[int, dict] = {}
        self.step_sids: List[int] = []                       # sequence of every row of the step that is running (set by the engine)
        self.stats = {"demoted_pages": 0, "cold_rows_fetched": 0, "bytes_h2d": 0, "bytes_d2h": 0, "materialised_layers": 0}

    # ------------------------------------------------------------------ sequences
    def on_create(self, sid: int):
        self.tier.create(sid)
        self.cold_map[sid] = torch.full((self.eng.max_pages,), -1, dtype=torch.int32)
        self.next_page[sid] = 0

    def on_free(self, sid: int):
        if sid in self.cold_map:
            self.tier.destroy(sid)
            del self.cold_map[sid], self.next_page[sid]

    def has_cold(self, sid: int) -> bool:
        return self.next_page.get(sid, 0) > 0

    def step_has_cold(self, R: int) -> bool:
        """Whether any row of the running step belongs to a sequence with pages in the cold tier."""
        return any(self.has_cold(sid) for sid in self.step_sids[:R])

    # ------------------------------------------------------------------ demotion
    def slide_window(self, sid: int) -> int:
        """Demote every page of the sequence that lies completely behind the hot window.  Returns the HBM pages released."""
        eng, m = self.eng, self.model
        s = eng.seqs[sid]
        upto = max(0, (s.length - self.hot_window) // self.page)
        first = self.next_page[sid]
        if upto <= first:
            return 0
        if upto - first > self.tier.free_cold_slots():
            raise RuntimeError(f"cold KV pool full: {upto - first} pages to demote, {self.tier.free_cold_slots()} cold slots free")
        self.tier.demotion_candidates(sid, s.length)          # sizes the native per-sequence table
        moved = []
        with torch.cuda.stream(self.copy_stream):
            self.copy_stream.wait_stream(eng.stream)
            for lp in range(first, upto):
                cs = self.tier.demote(sid, lp)
                phys = s.pages[lp]
                for i, t in m.kv_cache.items():
                    self.cold_kv[i][cs].copy_(t[phys], non_blocking=True)
                moved.append((lp, cs))
        self.copy_stream.synchronize()                        # the copies have left the HBM pages: they can be handed back
        for lp, cs in moved:
            eng.pa.swap_out(s.slot, lp)
            self.cold_map[sid][lp] = cs
        s.pages = eng.pa.pages(s.slot)
        with torch.cuda.stream(eng.stream):
            eng._sync_block_table(s)
        self.next_page[sid] = upto
        n = len(moved)
        self.stats["demoted_pages"] += n
        self.stats["bytes_d2h"] += n * self.page * self.rb * len(m.kv_cache)
        return n

    # ------------------------------------------------------------------ per-layer materialisation
    def _buf(self, R: int, sel_ld: int) -> dict:
        if R not in self._bufs:
            dev = self.model.device
            pm = (sel_ld + self.page - 1) // self.page
            b = {"pm": pm, "rows": pm * self.page,
                 "cache": torch.zeros(R * pm, self.page, self.rb, dtype=torch.uint8, device=dev),
                 "bt": torch.zeros(R, pm, dtype=torch.int32, device=dev), "seq": torch.zeros(R, dtype=torch.int32, device=dev),
                 "sel": torch.zeros(R, sel_ld, dtype=torch.int32, device=dev)}
            nat.call("lsb_kv_rows_identity", b["sel"], sel_ld, b["bt"], pm, b["seq"], R)
            self._bufs[R] = b
        return self._bufs[R]

    def materialise(self, layer: int, ws, R: int, sel_idx: torch.Tensor, sel_cnt: torch.Tensor, sel_ld: int):
        """Dense copy of the rows row r of the step attends to.  Returns (cache, block_table, max_pages, row_seq, sel_idx) to run the
        attention kernel with (``sel_cnt`` stays as it is)."""
        m = self.model
        b = self._buf(R, sel_ld)
        nat.call("lsb_kv_row_gather", m.kv_cache[layer], m.block_table, m.max_pages, ws.row_seq, sel_idx, sel_cnt, sel_ld, b["cache"], b["rows"],
                 R, self.page, self.rb)
        self.stats["materialised_layers"] += 1
        if any(self.has_cold(sid) for sid in self.step_sids[:R]):
            if self.h_sel is None or self.h_sel.shape[0] < R or self.h_sel.shape[1] != sel_ld + 1:
                self.h_sel = torch.zeros(max(R, 8), sel_ld + 1, dtype=torch.int32).pin_memory()
            cur = torch.cuda.current_stream(m.device)
            self.h_sel[:R, :sel_ld].copy_(sel_idx[:R], non_blocking=True)
            self.h_sel[:R, sel_ld].copy_(sel_cnt[:R], non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(cur)
            ev.synchronize()                                  # the one host wait per tiered attention layer: which rows were selected?
            n = 0
            flat_cold = self.cold_kv[layer].view(-1, self.rb)
            for r in range(R):
                sid = self.step_sids[r]
                if not self.has_cold(sid):
                    continue
                cnt = int(self.h_sel[r, sel_ld])
                pos = self.h_sel[r, :cnt].long()
                cs = self.cold_map[sid][pos // self.page].long()
                mask = cs >= 0
                k = int(mask.sum())
                if k == 0:
                    continue
                if n + k > self.max_staged:
                    raise RuntimeError(f"step reads {n + k} cold KV rows in one layer, the staging buffer holds {self.max_staged}: "
                                       "prefill chunks must run with their context hot")
                rows = cs[mask] * self.page + pos[mask] % self.page
                torch.index_select(flat_cold, 0, rows, out=self.h_stage[n: n + k])
                self.h_dst[n: n + k] = (r * b["rows"] + torch.nonzero(mask).squeeze(1)).int()
                n += k
            if n:
                self.d_stage[:n].copy_(self.h_stage[:n], non_blocking=True)
                self.d_dst[:n].copy_(self.h_dst[:n], non_blocking=True)
                nat.call("lsb_kv_row_scatter", self.d_stage, self.d_dst, n, b["cache"], self.rb)
                self.stats["cold_rows_fetched"] += n
                self.stats["bytes_h2d"] += n * (self.rb + 4)
        return b["cache"], b["bt"], b["pm"], b["seq"], b["sel"]
