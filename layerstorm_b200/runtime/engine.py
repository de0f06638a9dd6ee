"""Step engine: sequences, paged-cache bookkeeping, step staging, CUDA-graph decode.

One ``Engine`` drives one ``DeviceModel`` on one GPU.  A step is a batch of rows (decode: one
row per sequence; prefill: a chunk of consecutive tokens of one sequence; verify: a few
consecutive rows).  All per-step inputs are packed into one pinned host buffer and copied
with a single cudaMemcpyAsync; decode steps replay a captured CUDA graph per batch size,
so the host issues one copy + one graph launch + one 4-byte readback per generated token.

This is the role of the reference's CommandDispatcher + attention driver + sequence table
(src/daemon/command_dispatcher.h, src/daemon/attention/{attention_driver,kv_metadata,
page_provision}.cpp) with the ring protocol collapsed into direct calls: the reference's own
measurements identified per-layer host round trips, not bandwidth, as the decode wall
(docs/DESIGN-REVISIONS.md:46-54).
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import torch

from ..models.config import ModelConfig
from ..models.device_model import DeviceModel, Workspace
from ..ops import _native as nat
from . import native as rt
from .native import KvPoolExhausted  # noqa: F401  (re-exported: no free KV pages, the reference's kKvPoolExhausted)


class DeviceWaitError(RuntimeError):
    """A bounded device-side wait gave up during the step (a peer's flag never arrived, a tensor-core pipeline barrier never
    flipped): the step's output was computed from partial data and is withheld.  ``source`` names the error word
    ("tp_allreduce", "argmax_exchange", "context_parallel", "tensor_core"), ``code`` is the recorded value
    (collectives: 100 + the rank whose contribution was missing).  The word is sticky until :meth:`Engine.clear_device_errors`."""

    def __init__(self, source: str, code: int):
        super().__init__(f"device wait timed out: {source} error word = {code}" + (f" (rank {code - 100} did not arrive)" if code >= 100 else ""))
        self.source, self.code = source, code


def raise_on_error_words(names, values) -> None:
    """Host half of the per-step error check: ``values[i]`` is the error word read back for source ``names[i]``."""
    for name, v in zip(names, values):
        if int(v) != 0:
            raise DeviceWaitError(name, int(v))


@dataclass
class SequenceState:
    slot: int
    length: int = 0                 # tokens whose KV / recurrent state is committed
    pages: List[int] = field(default_factory=list)
    tokens: List[int] = field(default_factory=list)


@dataclass
class SamplingParams:
    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 1.0
    seed: int = 0
    max_tokens: int = 16


class Engine:
    def __init__(self, model: DeviceModel, max_seqs: int = 4, max_ctx: int = 4096, prefill_chunk: int = 256,
                 max_batch: int = 4, num_pages: Optional[int] = None, use_graph: bool = True, row_tiering: Optional[dict] = None):
        """``row_tiering``: ``{"hot_window_tokens": n, "cold_pages": m}`` keeps only the last n tokens of every sequence in HBM pages;
        older pages move to pinned host memory and single rows come back when the indexer selects them (eager steps, sparse-attention
        models; see runtime/kv_tiering.py).  ``num_pages`` can then be far below ``max_seqs * max_ctx / page``."""
        self.model, self.cfg = model, model.cfg
        if row_tiering:
            model.idx_identity = True                      # before the caches are allocated: indexer keys stay resident
        self.dev = model.device
        self.page = model.page
        self.max_ctx = max_ctx
        self.max_pages = (max_ctx + self.page - 1) // self.page
        self.num_pages = num_pages if num_pages is not None else self.max_pages * max_seqs
        self.max_seqs, self.max_batch, self.prefill_chunk = max_seqs, max_batch, prefill_chunk
        model.alloc_cache(self.num_pages, max_seqs, self.max_pages)
        self.pa = rt.PageAllocator([self.num_pages], self.page)
        self.free_slots = list(range(max_seqs - 1, -1, -1))
        self.seqs: Dict[int, SequenceState] = {}
        self.use_graph = use_graph and self.dev.type == "cuda"
        self.ws_decode: Dict[int, Workspace] = {}
        self.ws_prefill: Optional[Workspace] = None
        self.graphs: Dict[int, torch.cuda.CUDAGraph] = {}
        self.graph_launches: Dict[int, int] = {}
        Rmax = max(prefill_chunk, max_batch)
        self.h_bt = torch.zeros(max_seqs, self.max_pages, dtype=torch.int32).pin_memory()
        self.h_out = torch.zeros(Rmax, dtype=torch.int32).pin_memory()
        self.stream = torch.cuda.Stream(device=self.dev)
        self.row_tier = None
        if row_tiering:
            from .kv_tiering import RowTiering
            self.row_tier = RowTiering(self, int(row_tiering["hot_window_tokens"]), int(row_tiering["cold_pages"]))
            model.row_tier = self.row_tier
            self.use_graph = False                         # a tiered attention layer has a host round trip: eager steps
        self.vram_plan = self._carve_report()
        self.h_err = torch.zeros(8, dtype=torch.int32).pin_memory()      # error words of the step, read back with the sampled tokens
        self.h2d_bytes = 0
        self.d2h_bytes = 0
        self.kernel_launches = 0
        self.mtp = None               # MtpRunner once enable_mtp() was called (runtime/mtp.py)
        self.aux_listener = None      # object with on_rows / on_rewind / on_fork / on_free once enable_aux_capture() was called

    # ------------------------------------------------------------------ boot-time memory carve
    def _carve_report(self) -> dict:
        """The GPU's memory as the native planner carves it for what this engine has just allocated (weights, KV pages, indexer
        pages, recurrent state, step workspaces, expert slots): logged once at boot and kept as ``engine.vram_plan``.  The planner
        raises when a region does not fit, which turns an allocation that only succeeded by eating the safety margin into a
        visible boot error.  Reference: VramAllocator's boot carve log (src/core/memory/vram_allocator.h:19)."""
        import logging
        m, cfg = self.model, self.cfg
        if self.dev.type != "cuda":
            return {}
        free_b, total_b = torch.cuda.mem_get_info(self.dev)
        kv_page = sum(t[0].numel() * t.element_size() for t in m.kv_cache.values())
        idx_page = sum(t[0].numel() * t.element_size() for t in m.idx_cache.values())
        rec_seq = sum(t[0].numel() * t.element_size() for t in list(m.kda_state.values()) + list(m.kda_conv.values()) + list(m.idx_tail.values()))
        arenas = [L["arena"] for L in m.layers if L.get("arena") is not None]
        slot_b = arenas[0].ef.stride if arenas else 0
        slots = sum(a.n_slots for a in arenas)
        weights = m.weight_bytes() - slot_b * slots
        try:
            plan = rt.vram_plan(total_b, weights, workspace_bytes=256 << 20, kv_bytes_per_page=kv_page, kv_pages=self.num_pages, spec_pool_fraction=0.0,
                                indexer_bytes_per_page=idx_page, indexer_pages=self.num_pages if idx_page else 0,
                                recurrent_bytes_per_seq=rec_seq, recurrent_seqs=self.max_seqs, expert_slot_bytes=slot_b, expert_slots_wanted=slots,
                                stable_zone_fraction=1.0, safety_bytes=256 << 20)
        except rt.NativeError as e:
            logging.getLogger("layerstorm_b200.engine").warning("VRAM carve: %s (device has %.1f GiB, %.1f GiB free after allocation)",
                                                                e, total_b / 2 ** 30, free_b / 2 ** 30)
            return {"error": str(e)}
        plan["free_after_alloc_bytes"], plan["total_bytes"] = free_b, total_b
        gib = {k: round(v["size"] / 2 ** 30, 2) for k, v in plan["regions"].items() if v["size"]}
        logging.getLogger("layerstorm_b200.engine").info("VRAM carve (GiB): %s; %d KV pages of %d tokens, %d expert slots, %.1f GiB free",
                                                         gib, self.num_pages, self.page, plan["expert_stable_slots"], free_b / 2 ** 30)
        return plan

    # ------------------------------------------------------------------ device error words
    def _error_sources(self):
        """(name, int32 tensor view of one word) for every bounded-wait error word the model's kernels can set."""
        from ..models.device_model import TcScratch
        m = self.model
        src = [("tensor_core", TcScratch.get(self.dev).err[0:1])]
        if getattr(m, "comm", None) is not None:
            src.append(("tp_allreduce", m.comm.local_state[2:3]))
        if getattr(m, "comm_amax", None) is not None:
            src.append(("argmax_exchange", m.comm_amax.local_state[2:3]))
        dcp = getattr(m, "dcp", None)
        if dcp is not None and hasattr(dcp, "error_word"):
            src.append(("context_parallel", dcp.error_word()))
        return src

    def _queue_error_readback(self):
        """Called on the engine stream before the step's synchronize: the error words travel in the same device->host batch
        as the sampled tokens (4 bytes each)."""
        self._err_names = []
        for j, (name, t) in enumerate(self._error_sources()):
            self.h_err[j: j + 1].copy_(t, non_blocking=True)
            self._err_names.append(name)
        self.d2h_bytes += 4 * len(self._err_names)

    def _check_errors(self):
        raise_on_error_words(self._err_names, self.h_err[: len(self._err_names)].tolist())

    def clear_device_errors(self):
        """Reset the sticky error words after the cause (a dead or late rank) has been dealt with."""
        with torch.cuda.stream(self.stream):
            for _, t in self._error_sources():
                t.zero_()
        self.stream.synchronize()

    # ------------------------------------------------------------------ sequences
    def create_sequence(self) -> int:
        if not self.free_slots:
            raise RuntimeError("no free sequence slot")
        slot = self.free_slots.pop()
        self.seqs[slot] = SequenceState(slot)
        self.pa.create(slot)
        if self.row_tier is not None:
            self.row_tier.on_create(slot)
        with torch.cuda.stream(self.stream):
            self.model.reset_slot(slot)
        if self.mtp is not None:
            self.mtp.on_create(slot)
        return slot

    def free_sequence(self, sid: int):
        if getattr(self, "spilled", None) and sid in self.spilled:
            path, _ = self.spilled.pop(sid)
            try:
                os.remove(path)
            except OSError:
                pass
        if getattr(self, "hibernated", None) and sid in self.hibernated:
            self.hibernated.pop(sid)
            self.tier.destroy(sid)
        s = self.seqs.pop(sid)
        if self.mtp is not None:
            self.mtp.on_free(sid)
        if self.aux_listener is not None:
            self.aux_listener.on_free(sid)
        if self.row_tier is not None:
            self.row_tier.on_free(sid)
        self.pa.destroy(s.slot)
        self.free_slots.append(s.slot)

    def free_page_count(self) -> int:
        return self.pa.free_pages(0)

    def configure_expert_cache(self, section: dict) -> bool:
        """Apply the ``memory.expert_cache`` eviction policy and weights to the capped expert cache, if this engine streams experts
        (live-changeable; mirrored to every rank of a multi-process server).  Returns whether a cache took them."""
        streamer = getattr(self.model, "streamer", None)
        if streamer is None:
            return False
        streamer.configure_eviction(section)
        return True

    def seq_len(self, sid: int) -> int:
        return self.seqs[sid].length

    @property
    def has_recurrent_state(self) -> bool:
        return any(self.cfg.is_kda_layer(i) for i in range(self.cfg.n_layers))

    def fork_sequence(self, parent: int, prefix_len: Optional[int] = None) -> int:
        """Truncating fork: the child shares the parent's KV pages covering ``prefix_len`` tokens
        (reference counted, copy-on-write on the frontier page).  Recurrent (KDA) state cannot be
        rolled back, so models with KDA layers only fork at the parent's full length."""
        if getattr(self.model, "dcp", None) is not None:
            raise NotImplementedError("not available with a sharded KV cache")
        self._require_hot(parent)                 # a hibernated / spilled holder comes back to HBM before its pages are shared
        ps = self.seqs[parent]
        prefix_len = ps.length if prefix_len is None else prefix_len
        has_kda = any(self.cfg.is_kda_layer(i) for i in range(self.cfg.n_layers))
        if has_kda and prefix_len != ps.length:
            raise RuntimeError("a sequence with recurrent state can only be forked at its frontier")
        if self.cfg.index_kpool > 1 and prefix_len % self.cfg.index_kpool and prefix_len != ps.length:
            raise RuntimeError("fork point must be a multiple of the indexer pool size")
        if not self.free_slots:
            raise RuntimeError("no free sequence slot")
        slot = self.free_slots.pop()
        self.pa.fork(ps.slot, slot, prefix_len)
        cs = SequenceState(slot, length=prefix_len, pages=self.pa.pages(slot), tokens=list(ps.tokens[:prefix_len]))
        self.seqs[slot] = cs
        with torch.cuda.stream(self.stream):
            m = self.model
            for t in list(m.kda_state.values()) + list(m.kda_conv.values()) + list(m.idx_tail.values()):
                t[slot].copy_(t[ps.slot])
            self._sync_block_table(cs)
            if self.mtp is not None:
                self.mtp.on_fork(parent, slot, prefix_len)
            if self.aux_listener is not None:
                self.aux_listener.on_fork(parent, slot, prefix_len)
        return slot

    # ------------------------------------------------------------------ KV tiering (hibernate / resume)
    def enable_kv_tiering(self, cold_pages: int):
        """Reserve a pinned host pool of ``cold_pages`` KV pages (all attention layers of a page travel together).
        A hibernated sequence gives its HBM pages back to the pool and keeps only host copies; its slot (recurrent
        state, indexer tail) stays.  The native tier table tracks which logical page sits in which cold slot."""
        m = self.model
        self.cold_pages = cold_pages
        self.tier = rt.KvTierTable(self.page, 0, cold_pages, 0)
        self.cold_kv = {i: torch.empty(cold_pages, *t.shape[1:], dtype=t.dtype).pin_memory() for i, t in m.kv_cache.items()}
        self.cold_idx = {i: torch.empty(cold_pages, *t.shape[1:], dtype=t.dtype).pin_memory() for i, t in m.idx_cache.items()}
        self.hibernated: Dict[int, List[int]] = {}
        self.copy_stream = torch.cuda.Stream(device=self.dev)

    def hibernate(self, sid: int) -> int:
        """Move every KV page of the sequence to pinned host memory and free its HBM pages.  Returns the pages freed.
        Shared (forked) pages are copied too: the sequence becomes independent of its relatives."""
        if getattr(self.model, "dcp", None) is not None:
            raise NotImplementedError("not available with a sharded KV cache")
        s = self.seqs[sid]
        if self.row_tier is not None:
            raise NotImplementedError("whole-sequence hibernation and row-granular tiering are alternatives: this engine tiers rows")
        if sid in self.hibernated:
            return 0
        n = len(s.pages)
        if n > self.tier.free_cold_slots():
            raise RuntimeError(f"cold pool full: need {n} pages, {self.tier.free_cold_slots()} free")
        self.tier.create(sid)
        self.tier.demotion_candidates(sid, n * self.page + self.page)          # sizes the per-sequence table
        slots = [self.tier.demote(sid, p) for p in range(n)]
        self.stream.synchronize()                                              # the pages are final
        with torch.cuda.stream(self.copy_stream):
            for p, (pg, cs) in enumerate(zip(s.pages, slots)):
                for i, t in self.model.kv_cache.items():
                    self.cold_kv[i][cs].copy_(t[pg], non_blocking=True)
                for i, t in self.model.idx_cache.items():
                    self.cold_idx[i][cs].copy_(t[pg], non_blocking=True)
            self.d2h_bytes += n * sum(t[0].numel() * t.element_size() for t in list(self.model.kv_cache.values()) + list(self.model.idx_cache.values()))
        self.copy_stream.synchronize()
        self.pa.rewind(s.slot, 0)                                              # HBM pages go back to the allocator
        self.hibernated[sid] = slots
        s.pages = []
        return n

    def resume(self, sid: int):
        """Bring a hibernated sequence back: allocate pages, copy host -> device, rebuild the block table."""
        slots = self.hibernated[sid]
        s = self.seqs[sid]
        self.pa.extend(s.slot, s.length)                                       # may raise KvPoolExhausted: the caller evicts and retries
        self.hibernated.pop(sid)                                               # only now: a failed extend leaves the sequence hibernated, cold slots intact
        s.pages = self.pa.pages(s.slot)
        with torch.cuda.stream(self.copy_stream):
            for pg, cs in zip(s.pages, slots):
                for i, t in self.model.kv_cache.items():
                    t[pg].copy_(self.cold_kv[i][cs], non_blocking=True)
                for i, t in self.model.idx_cache.items():
                    t[pg].copy_(self.cold_idx[i][cs], non_blocking=True)
            self.h2d_bytes += len(slots) * sum(t[0].numel() * t.element_size() for t in list(self.model.kv_cache.values()) + list(self.model.idx_cache.values()))
        self.copy_stream.synchronize()
        self.tier.destroy(sid)
        with torch.cuda.stream(self.stream):
            self._sync_block_table(s)

    # ------------------------------------------------------------------ second tiering hop: hibernated sequence -> file
    def spill(self, sid: int, path: str) -> int:
        """Write a HIBERNATED sequence's cold KV (and indexer) pages to ``path`` and give its pinned host slots back.  Returns the
        bytes written.  The file is a cache entry, not a store: ``unspill`` raises when it is gone or damaged and the caller drops
        the sequence.  Reference: CMD_SEQ_HIBERNATE spill=1 (python/orchestrator/orchestrator.py:455-484, the engine owns the byte moves)."""
        import json
        import struct
        if sid not in getattr(self, "hibernated", {}):
            raise RuntimeError("only a hibernated sequence can be spilled")
        slots = self.hibernated[sid]
        s = self.seqs[sid]
        parts = [(("kv", i), t) for i, t in sorted(self.cold_kv.items())] + [(("idx", i), t) for i, t in sorted(self.cold_idx.items())]
        head = json.dumps({"version": 1, "length": s.length, "pages": len(slots), "page": self.page,
                           "tensors": [[k[0], k[1], list(t.shape[1:]), str(t.dtype)] for k, t in parts]}).encode()
        idx = torch.tensor(slots, dtype=torch.long)
        nbytes = 0
        tmp = path + ".tmp"
        with open(tmp, "wb") as fh:
            fh.write(b"LSBSPILL" + struct.pack("<I", len(head)) + head)
            for _, t in parts:
                blob = t[idx].contiguous().view(torch.uint8).numpy().tobytes() if len(slots) else b""
                fh.write(blob)
                nbytes += len(blob)
        os.replace(tmp, path)
        self.tier.destroy(sid)                                                 # the pinned slots are free again
        self.hibernated.pop(sid)
        if not hasattr(self, "spilled"):
            self.spilled: Dict[int, tuple] = {}
        self.spilled[sid] = (path, len(slots))
        return nbytes

    def unspill(self, sid: int):
        """Read a spilled sequence back into pinned host slots (it is then hibernated again; ``resume`` brings it to HBM).  Raises
        OSError / ValueError when the file is missing, truncated or does not match this engine's cache geometry."""
        import json
        import struct
        path, n = self.spilled[sid]
        parts = [(("kv", i), t) for i, t in sorted(self.cold_kv.items())] + [(("idx", i), t) for i, t in sorted(self.cold_idx.items())]
        with open(path, "rb") as fh:
            if fh.read(8) != b"LSBSPILL":
                raise ValueError(f"{path}: not a spill file")
            (hl,) = struct.unpack("<I", fh.read(4))
            head = json.loads(fh.read(hl))
            want = [[k[0], k[1], list(t.shape[1:]), str(t.dtype)] for k, t in parts]
            if head.get("pages") != n or head.get("page") != self.page or head.get("tensors") != want or head.get("length") != self.seqs[sid].length:
                raise ValueError(f"{path}: written for another cache geometry or sequence")
            if n > self.tier.free_cold_slots():
                raise RuntimeError(f"cold pool full: need {n} pages, {self.tier.free_cold_slots()} free")
            blobs = []
            for _, t in parts:
                per = t[0].numel() * t.element_size()
                b = fh.read(n * per)
                if len(b) != n * per:
                    raise ValueError(f"{path}: truncated")
                blobs.append(b)
        self.tier.create(sid)
        self.tier.demotion_candidates(sid, n * self.page + self.page)
        slots = [self.tier.demote(sid, p) for p in range(n)]
        idx = torch.tensor(slots, dtype=torch.long)
        for (_, t), b in zip(parts, blobs):
            if n:
                t[idx] = torch.frombuffer(bytearray(b), dtype=torch.uint8).view(t.dtype).view(n, *t.shape[1:])
        self.hibernated[sid] = slots
        self.spilled.pop(sid)

    def _require_hot(self, sid: int):
        if getattr(self, "spilled", None) and sid in self.spilled:
            self.unspill(sid)
        if getattr(self, "hibernated", None) and sid in self.hibernated:
            self.resume(sid)

    def _copy_page(self, src: int, dst: int):
        m = self.model
        for t in list(m.kv_cache.values()) + list(m.idx_cache.values()):
            t[dst].copy_(t[src])

    def _sync_block_table(self, s: SequenceState):
        for j, pg in enumerate(s.pages):
            self.h_bt[s.slot, j] = pg
        self.model.block_table[s.slot].copy_(self.h_bt[s.slot], non_blocking=True)
        self.h2d_bytes += self.max_pages * 4

    # ------------------------------------------------------------------ recurrent-state anchors
    def anchor(self, sid: int):
        """Snapshot the recurrent state of a sequence (KDA state and convolution history, the indexer's open-pool tail) at its
        current frontier.  ``rewind`` to a later-or-equal position restores the snapshot and replays the tokens after it, which is
        how a partly rejected speculative round is undone on models whose state cannot be un-applied (the reference's KDA anchor
        snapshot / restore, src/daemon/ipc_protocol.h:214-216).  One anchor per engine (requests are served one at a time)."""
        s = self.seqs[sid]
        m = self.model
        if not hasattr(self, "_anchor_buf"):
            self._anchor_buf = {"state": {i: torch.empty_like(t[0]) for i, t in m.kda_state.items()},
                                "conv": {i: torch.empty_like(t[0]) for i, t in m.kda_conv.items()},
                                "tail": {i: torch.empty_like(t[0]) for i, t in m.idx_tail.items()}}
        with torch.cuda.stream(self.stream):
            for key, src in (("state", m.kda_state), ("conv", m.kda_conv), ("tail", m.idx_tail)):
                for i, t in src.items():
                    self._anchor_buf[key][i].copy_(t[s.slot], non_blocking=True)
        self._anchor_of = (sid, s.length)

    def _restore_anchor(self, s: SequenceState):
        m = self.model
        for key, dst in (("state", m.kda_state), ("conv", m.kda_conv), ("tail", m.idx_tail)):
            for i, t in dst.items():
                t[s.slot].copy_(self._anchor_buf[key][i], non_blocking=True)

    def _ws_rows(self, R: int) -> Workspace:
        """Cached workspace for verify / replay steps of R consecutive rows of one sequence (logits for every row)."""
        if not hasattr(self, "ws_verify"):
            self.ws_verify: Dict[int, Workspace] = {}
        if R not in self.ws_verify:
            self.ws_verify[R] = Workspace(self.model, R, R, self.max_ctx)
        return self.ws_verify[R]

    def rewind(self, sid: int, length: int):
        """Roll the committed frontier back (speculative-verify rejection).  Models with recurrent (KDA) state need an anchor
        taken at or before ``length`` (:meth:`anchor`): the state is restored from it and the tokens between the anchor and
        ``length`` are replayed."""
        if getattr(self.model, "dcp", None) is not None:
            raise NotImplementedError("not available with a sharded KV cache")
        s = self.seqs[sid]
        if length == s.length:
            return
        if self.row_tier is not None and length < self.row_tier.next_page.get(sid, 0) * self.page:
            raise RuntimeError("rewind into the cold part of a tiered sequence is refused")
        replay: List[int] = []
        if self.has_recurrent_state and length < s.length:
            a_sid, a_len = getattr(self, "_anchor_of", (None, -1))
            if a_sid != sid or a_len > length or a_len < 0:
                raise RuntimeError("rewind of a recurrent-state sequence needs an anchor at or before the target position")
            replay = list(s.tokens[a_len:length])
            length_after = length
            length = a_len
            with torch.cuda.stream(self.stream):
                self._restore_anchor(s)
        s.length = length
        del_tokens = s.tokens[length:]
        del s.tokens[length:]
        if self.mtp is not None:
            self.mtp.on_rewind(sid, length)
        if self.aux_listener is not None:
            self.aux_listener.on_rewind(sid, length)
        self.pa.rewind(s.slot, length)
        s.pages = self.pa.pages(s.slot)
        if replay:
            # teacher-forced replay of the accepted tokens rebuilds the recurrent state (and rewrites the same KV rows)
            self.forward_rows(sid, replay, commit=True, want_logits=False)
            assert s.length == length_after
        del del_tokens

    def _ensure_pages(self, s: SequenceState, new_len: int):
        if (new_len + self.page - 1) // self.page > self.max_pages:
            raise RuntimeError(f"sequence length {new_len} exceeds max context {self.max_ctx}")
        cow = self.pa.cow_frontier(s.slot)          # shared frontier page must become private first
        if cow is not None:
            self._copy_page(*cow)
        dcp = getattr(self.model, "dcp", None)
        if dcp is not None:
            # sharded KV: a rank stores only its share of the positions.  Every rank pages for the LARGEST share (rank 0's, at most
            # one chunk more than its own), so that the allocators of all ranks stay in the same state and a pool-exhausted error
            # is raised by every rank in the same call - the ranks of a multi-process server must fail together or not at all
            from ..parallel.dcp import local_length
            new_len = local_length(new_len, dcp.chunk, dcp.world, 0)
        new = self.pa.extend(s.slot, new_len)
        if new or cow is not None:
            s.pages = self.pa.pages(s.slot)
            self._sync_block_table(s)

    # ------------------------------------------------------------------ staging
    def _stage(self, ws: Workspace, rows: List[tuple], seq_groups: List[tuple]):
        """rows: (token, slot, pos); seq_groups: (row0, nrows, slot)."""
        R = len(rows)
        P = max(self.cfg.index_kpool, 1)
        if self.row_tier is not None:
            self.row_tier.step_sids = [slot for (_, slot, _) in rows]      # sequence id == slot id in this engine
        # ring of pinned staging buffers: a buffer is rewritten only after the copy that last
        # read it has completed, so the host can run ahead of the device by several steps
        if not hasattr(ws, "h_ring"):
            ws.h_ring = [torch.zeros(9, ws.R, dtype=torch.int32).pin_memory() for _ in range(4)]
            ws.h_ev = [None] * 4
            ws.h_i = 0
        k = ws.h_i
        ws.h_i = (k + 1) % 4
        if ws.h_ev[k] is not None:
            ws.h_ev[k].synchronize()
        h = ws.h_ring[k]
        h.zero_()
        h[1].fill_(-1)
        for r, (tok, slot, pos) in enumerate(rows):
            h[0, r] = tok; h[1, r] = slot; h[2, r] = pos; h[3, r] = pos + 1; h[4, r] = slot
            h[5, r] = (pos + 1) // P
        for j, (r0, n, slot) in enumerate(seq_groups):
            h[6, j] = r0; h[7, j] = n; h[8, j] = slot
        # host-side facts about the step that size kernels' grids: the largest index-entry count of a row, one sequence or several
        ws.ne_hint = max((pos + 1) // P for (_, _, pos) in rows) if rows else 0
        ws.single_seq = len(seq_groups) == 1 and len({slot for (_, slot, _) in rows}) == 1
        ws.inp.copy_(h, non_blocking=True)
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream())
        ws.h_ev[k] = ev
        self.h2d_bytes += 9 * ws.R * 4

    def _ws_decode(self, B: int) -> Workspace:
        if B not in self.ws_decode:
            self.ws_decode[B] = Workspace(self.model, B, B, self.max_ctx)
        return self.ws_decode[B]

    # ------------------------------------------------------------------ steps
    def prefill(self, sid: int, tokens: Sequence[int], want_logits: bool = False):
        """Append ``tokens`` to the sequence in chunks; returns the greedy next token (and the
        last-position logits when asked)."""
        self._require_hot(sid)
        s = self.seqs[sid]
        tokens = [int(t) for t in tokens]
        if self.ws_prefill is None:
            self.ws_prefill = Workspace(self.model, self.prefill_chunk, 1, self.max_ctx)
        ws = self.ws_prefill
        nxt, logits = None, None
        if self.mtp is not None and tokens:
            self.mtp.before_step(sid, tokens[0])
        with torch.cuda.stream(self.stream):
            # all pages of the call up front: running out of pages must fail BEFORE the first chunk is committed, because the
            # caller evicts and calls again with the same tokens (a failure after chunk c would append chunks 0..c twice)
            self._ensure_pages(s, s.length + len(tokens))
            for c0 in range(0, len(tokens), self.prefill_chunk):
                chunk = tokens[c0: c0 + self.prefill_chunk]
                R = len(chunk)
                rows = [(t, s.slot, s.length + j) for j, t in enumerate(chunk)]
                self._stage(ws, rows, [(0, R, s.slot)])
                n0 = nat.launch_count()
                self.model.forward(ws, R, 1, R - 1, 1)
                self.model.argmax(ws, 1)
                if self.mtp is not None:
                    self.mtp.after_prefill_chunk(sid, ws, chunk, s.length, tokens[c0 + R] if c0 + R < len(tokens) else None)
                if self.aux_listener is not None:
                    self._aux_rows(sid, 0, R, s.length, chunk)
                self.kernel_launches += nat.launch_count() - n0
                s.length += R
                s.tokens.extend(chunk)
            self.h_out[:1].copy_(ws.out_tok[:1], non_blocking=True)
            self.d2h_bytes += 4
            self._queue_error_readback()
            self.stream.synchronize()
            self._check_errors()
            nxt = int(self.h_out[0])
            if want_logits:
                logits = ws.logits[0].float().cpu()
            if self.mtp is not None:
                self.mtp.release_pins()
        if self.row_tier is not None:
            self.row_tier.slide_window(sid)
        return (nxt, logits) if want_logits else nxt

    def sample_last_prefill(self, sid: int, sample) -> int:
        """Draw the first generated token of a sampled request from the logits the sequence's prefill left in the prefill
        workspace (the last prompt position), on the device."""
        ws = self.ws_prefill
        s = self.seqs[sid]
        temperature, top_k, top_p, seed = sample
        with torch.cuda.stream(self.stream):
            offs = torch.tensor([s.length - 1], dtype=torch.int64, device=self.dev)
            nat.call("lsb_sample", ws.logits, ws.logits.shape[1], 1, ws.logits.shape[1], float(temperature), int(top_k), float(top_p),
                     int(seed) & 0x7FFFFFFFFFFFFFFF, offs, ws.out_tok)
            self.h_out[:1].copy_(ws.out_tok[:1], non_blocking=True)
            self.d2h_bytes += 4
            self.stream.synchronize()
        return int(self.h_out[0])

    def forward_rows(self, sid: int, tokens: Sequence[int], commit: bool = True, want_logits: bool = True) -> Optional[torch.Tensor]:
        """Run consecutive rows of one sequence and return logits for ALL rows (verify shape)."""
        self._require_hot(sid)
        s = self.seqs[sid]
        R = len(tokens)
        if self.mtp is not None and R:
            self.mtp.before_step(sid, int(tokens[0]))
        ws = self._ws_rows(R)
        with torch.cuda.stream(self.stream):
            self._ensure_pages(s, s.length + R)
            rows = [(int(t), s.slot, s.length + j) for j, t in enumerate(tokens)]
            self._stage(ws, rows, [(0, R, s.slot)])
            n0 = nat.launch_count()
            self.model.forward(ws, R, 1, 0, R)
            self.kernel_launches += nat.launch_count() - n0
            if self.mtp is not None:
                self.mtp.stash_rows(sid, ws, 0, R, s.length)
            if self.aux_listener is not None and commit:
                self._aux_rows(sid, 0, R, s.length, tokens)
            self._queue_error_readback()
            self.stream.synchronize()
            self._check_errors()
        if commit:
            s.length += R
            s.tokens.extend(int(t) for t in tokens)
        else:
            self.pa.rewind(s.slot, s.length)
            s.pages = self.pa.pages(s.slot)
        if not want_logits:
            return None
        self.d2h_bytes += R * ws.logits.shape[1] * 4
        return ws.logits[:R].float().cpu()

    def verify_greedy(self, sid: int, tok: int, draft: Sequence[int]):
        """One speculative round decided on the device: feeds ``[tok] + draft`` as consecutive rows, takes the target's arg-max at
        every row, counts the agreeing draft prefix with ``lsb_spec_verify`` and reads back 8 bytes: (accepted draft tokens, the
        target's own next token).  ``tok`` and the accepted tokens are committed; on a partial acceptance the rest is rolled back
        (recurrent models: anchor + replay).  Returns ``(n_accepted, next_token)``."""
        self._require_hot(sid)
        s = self.seqs[sid]
        draft = [int(t) for t in draft]
        rows_tok = [int(tok)] + draft
        R, gamma = len(rows_tok), len(draft)
        if self.mtp is not None:
            self.mtp.before_step(sid, int(tok))
        ws = self._ws_rows(R)
        if not hasattr(ws, "verify_out"):
            ws.verify_out = torch.zeros(2, dtype=torch.int32, device=self.dev)
        ca = getattr(self.model, "comm_amax", None)
        if ca is not None and 2 * R > ca.cap:
            raise RuntimeError(f"the arg-max exchange buffer holds {ca.cap // 2} rows, the verify step has {R}")
        if self.has_recurrent_state and gamma > 0:
            self.anchor(sid)
        with torch.cuda.stream(self.stream):
            self._ensure_pages(s, s.length + R)
            rows = [(t, s.slot, s.length + j) for j, t in enumerate(rows_tok)]
            self._stage(ws, rows, [(0, R, s.slot)])
            n0 = nat.launch_count()
            self.model.forward(ws, R, 1, 0, R)
            self.model.argmax(ws, R)
            # rows 1..gamma of the staged token ids ARE the draft; out_tok[k] is the target's choice after row k
            nat.call("lsb_spec_verify", ws.tok[1:] if gamma else ws.tok, ws.out_tok, gamma, ws.verify_out)
            self.kernel_launches += nat.launch_count() - n0
            if self.mtp is not None:
                self.mtp.stash_rows(sid, ws, 0, R, s.length)
            if self.aux_listener is not None:
                self._aux_rows(sid, 0, R, s.length, rows_tok)       # all rows; the rewind below takes the rejected ones back
            self.h_out[:2].copy_(ws.verify_out, non_blocking=True)
            self.d2h_bytes += 8
            self._queue_error_readback()
            self.stream.synchronize()
            self._check_errors()
        n_acc, nxt = int(self.h_out[0]), int(self.h_out[1])
        s.length += R
        s.tokens.extend(rows_tok)
        if n_acc < gamma:
            self.rewind(sid, s.length - (gamma - n_acc))
        return n_acc, nxt

    def enable_aux_capture(self, layer_ids, listener):
        """From now on every committed step hands the target's hidden states at ``layer_ids`` to ``listener``:
        ``listener.on_rows(sid, first_position, aux [rows, len(layer_ids) * hidden], tokens)`` right after the step's kernels were
        queued, on the engine's stream (the view is overwritten by the next step: the listener consumes it there and then), plus
        ``on_rewind(sid, length)``, ``on_fork(parent, child, prefix_len)`` and ``on_free(sid)``.  One GPU; steps that are not
        committed (``forward_rows(commit=False)``) are not reported.  Used by the block draft (``speculation/dspark.py``)."""
        if self.row_tier is not None or getattr(self.model, "dcp", None) is not None:
            raise NotImplementedError("aux hidden capture needs an untiered, unsharded KV cache")
        self.model.set_aux_capture(layer_ids, max(self.prefill_chunk, self.max_batch, 64))
        self.graphs.clear()                  # graphs captured so far do not contain the copies
        self.graph_launches.clear()
        self.aux_listener = listener

    def _aux_rows(self, sid: int, row0: int, n: int, pos0: int, tokens):
        buf = self.model.aux_capture["buf"]
        self.aux_listener.on_rows(sid, pos0, buf[row0: row0 + n].view(n, -1), tokens)

    def enable_mtp(self):
        """Keep the model's multi-token-prediction block in step with every sequence from now on (``runtime/mtp.py``) so that
        :meth:`mtp_draft` can propose a token; costs one pass of the block per committed token.  Raises NotImplementedError when
        the model has no block on the device or the engine's KV / expert placement rules it out."""
        if self.mtp is None:
            from .mtp import MtpRunner
            self.mtp = MtpRunner(self)
        return self.mtp

    def mtp_draft(self, sid: int, next_tok: int) -> List[int]:
        """The MTP block's proposal for the token AFTER ``next_tok`` (the token about to be fed to the sequence); [] when the
        block is not in step with the sequence.  Verify with :meth:`verify_greedy` ``(sid, next_tok, draft)``."""
        if self.mtp is None:
            raise RuntimeError("call enable_mtp() first")
        self._require_hot(sid)
        return self.mtp.draft(sid, int(next_tok))

    @property
    def supports_device_sampling(self) -> bool:
        """Whether ``decode(..., sample=...)`` can draw the next token on the device (needs the whole vocabulary on this GPU)."""
        return self.model.tp_size == 1

    def set_layer_skip(self, skip=(), probe: bool = False):
        """Draft-pass layer skipping (see ``DeviceModel.set_layer_skip``); applies to the following steps of this engine."""
        self.model.set_layer_skip(skip, probe)

    def layer_similarities(self) -> Dict[int, float]:
        """Per executed layer of the last probed step: cosine similarity between the layer's input and the next executed layer's input
        (one small D2H read; only while probing is on)."""
        pr = self.model.probe
        if pr is None:
            return {}
        with torch.cuda.stream(self.stream):
            v = pr["sims"].cpu()
        run = [i for i in range(self.cfg.n_layers) if i not in self.model.skip_layers]
        return {l: float(v[l]) for l in run[:-1]}

    @property
    def supports_confidence(self) -> bool:
        """Whether ``decode(confidence=True)`` can report the step's top-1 probability (the whole vocabulary on this GPU)."""
        return self.model.tp_size == 1

    def decode(self, sids: Sequence[int], tokens: Sequence[int], return_logits: bool = False, sample=None, confidence: bool = False):
        """One decode step for a batch of sequences: feeds ``tokens[i]`` at the frontier of
        ``sids[i]`` and returns the next token per sequence - the arg-max, or with ``sample = (temperature, top_k, top_p,
        seed)`` a draw from the filtered distribution made on the device (Philox stream keyed by the seed and the token's
        position, so a fixed seed reproduces the trajectory); either way only 4 bytes per row come back."""
        B = len(sids)
        for sid in sids:
            self._require_hot(sid)
        if self.mtp is not None:
            for sid, tok in zip(sids, tokens):
                self.mtp.before_step(sid, int(tok))
        ws = self._ws_decode(B)
        with torch.cuda.stream(self.stream):
            rows, groups = [], []
            for j, (sid, tok) in enumerate(zip(sids, tokens)):
                s = self.seqs[sid]
                self._ensure_pages(s, s.length + 1)
                rows.append((int(tok), s.slot, s.length))
                groups.append((j, 1, s.slot))
            self._stage(ws, rows, groups)
            if self.use_graph:
                # one graph per batch size and per set of skipped layers (a draft pass that leaves layers out replays its own graph)
                gk = B if not (self.model.skip_layers or self.model.probe is not None) else (B, self.model.skip_layers, self.model.probe is not None)
                if gk not in self.graphs:
                    if len(self.graphs) > 64:
                        raise RuntimeError("too many captured decode graphs (layer-skip sets): clear Engine.graphs")
                    self._capture(B, ws, gk)
                self.graphs[gk].replay()
                self.kernel_launches += self.graph_launches[gk]
            else:
                n0 = nat.launch_count()
                self.model.forward(ws, B, B, 0, B)
                self.model.argmax(ws, B)
                self.kernel_launches += nat.launch_count() - n0
            if self.mtp is not None:
                for j, sid in enumerate(sids):
                    self.mtp.stash_rows(sid, ws, j, 1, self.seqs[sid].length)
            if self.aux_listener is not None:
                for j, (sid, tok) in enumerate(zip(sids, tokens)):
                    self._aux_rows(sid, j, 1, self.seqs[sid].length, [int(tok)])
            if sample is not None:
                if not self.supports_device_sampling:
                    raise RuntimeError("device sampling needs the full vocabulary on one GPU")
                temperature, top_k, top_p, seed = sample
                offs = ws.row_pos[:B].to(torch.int64)
                nat.call("lsb_sample", ws.logits, ws.logits.shape[1], B, ws.logits.shape[1], float(temperature), int(top_k), float(top_p),
                         int(seed) & 0x7FFFFFFFFFFFFFFF, offs, ws.out_tok)
                self.kernel_launches += 1
            self.h_out[:B].copy_(ws.out_tok[:B], non_blocking=True)
            self.d2h_bytes += 4 * B
            if confidence:
                # top-1 probability and normalised entropy (H / ln V) of every row's distribution, computed on the device: 8 more bytes per row
                if not self.supports_confidence:
                    raise RuntimeError("step confidence needs the full vocabulary on one GPU")
                if not hasattr(ws, "conf"):
                    ws.conf = torch.zeros(2, ws.R, device=self.dev)
                    ws.h_conf = torch.zeros(2, ws.R).pin_memory()
                V = ws.logits.shape[1]
                nat.call("lsb_confidence", ws.logits, V, B, V, ws.conf[0], ws.conf[1])
                self.kernel_launches += 1
                ws.h_conf.copy_(ws.conf, non_blocking=True)
                self.d2h_bytes += 8 * B
            self._queue_error_readback()
            self.stream.synchronize()
            self._check_errors()
        out = [int(self.h_out[j]) for j in range(B)]
        if confidence:
            conf = [(float(ws.h_conf[0, j]), float(ws.h_conf[1, j])) for j in range(B)]
        for sid, tok in zip(sids, tokens):
            s = self.seqs[sid]
            s.length += 1
            s.tokens.append(int(tok))
            if self.row_tier is not None and s.length % self.page == 0:
                self.row_tier.slide_window(sid)
        if return_logits:
            return out, ws.logits[:B].float().cpu()
        if confidence:
            return out, conf
        return out

    def _capture(self, B: int, ws: Workspace, gk=None):
        gk = B if gk is None else gk
        # warm-up run outside capture (sets function attributes, touches every buffer); the KDA
        # state it perturbs is restored by snapshotting the affected slots first.
        slots = [int(ws.seq_slot[j]) for j in range(B)]
        snap = self._snapshot_recurrent(slots)
        self.model.forward(ws, B, B, 0, B)
        self.model.argmax(ws, B)
        self.stream.synchronize()
        self._restore_recurrent(slots, snap)
        g = torch.cuda.CUDAGraph()
        n0 = nat.launch_count()
        with torch.cuda.graph(g, stream=self.stream):
            self.model.forward(ws, B, B, 0, B)
            self.model.argmax(ws, B)
        self.graph_launches[gk] = nat.launch_count() - n0
        self._restore_recurrent(slots, snap)
        self.graphs[gk] = g

    def _snapshot_recurrent(self, slots):
        m = self.model
        return {"state": {i: t[slots].clone() for i, t in m.kda_state.items()},
                "conv": {i: t[slots].clone() for i, t in m.kda_conv.items()}}

    def _restore_recurrent(self, slots, snap):
        m = self.model
        for i, t in m.kda_state.items():
            t[slots] = snap["state"][i]
        for i, t in m.kda_conv.items():
            t[slots] = snap["conv"][i]

    # ------------------------------------------------------------------ user-facing
    def generate(self, prompt: Sequence[int], max_new_tokens: int = 16, eos: Optional[Sequence[int]] = None,
                 on_token=None) -> List[int]:
        """Greedy generation for one prompt (prefill + decode loop)."""
        sid = self.create_sequence()
        try:
            out = []
            tok = self.prefill(sid, prompt)
            for _ in range(max_new_tokens):
                out.append(tok)
                if on_token:
                    on_token(tok)
                if eos and tok in eos:
                    break
                tok = self.decode([sid], [tok])[0]
            return out
        finally:
            self.free_sequence(sid)
