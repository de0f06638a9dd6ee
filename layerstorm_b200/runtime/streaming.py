"""Capped VRAM expert cache backed by pinned host memory (expert streaming).

Each MoE layer keeps ``slots_per_layer`` expert slots in HBM; every expert's slot image lives in a
pinned host store.  Per layer and step:
  1. the routed expert ids come back to the host through a pinned buffer (the only host wait of the layer),
  2. missing experts are fetched host->device with pinned ``cudaMemcpyAsync`` on a side stream -
     what is fetched when is decided by the native ``TransferEngine`` (de-duplication, priorities,
     in-flight waterline) and where it lands by the native ``ExpertCache`` (impact-weighted LRU,
     locked while in use),
  3. the copies are gated on the DEVICE: the side stream records an event after the wave's copies, the compute stream
     waits for it (``cudaStreamWaitEvent``; the reference's ``record_h2d_barrier``, src/core/transfer/transfer_engine.h:159,223)
     and runs the expert kernels; the side stream in turn waits for the kernels' event before it overwrites a slot.  The host
     does not wait for a copy.  When a step needs more experts than the layer has slots (prefill chunks) this repeats in
     waves, and the combine runs once at the end.
With ``fetch_deadline_ms`` set, the host polls the wave's copy event up to the deadline; experts whose copies have not
landed by then are left out of this step (the step finishes DEGRADED, the combine skips their slots) and are ready for the
next one - the reference's deadline -> degraded -> retry (src/daemon/moe/moe_progressive.cpp:579-586).
Prefetch: the experts a step used at layer i are requested for layer i+1 at low priority while
layer i computes ("same-index" heuristic), and dropped if the router disagrees.
Reference behaviour: progressive FETCH_AND_RUN_MOE waves with an explicit evict map
(src/daemon/moe/moe_progressive.cpp:441-453), TransferEngine + ExpertCache + pinned arena.
"""
from __future__ import annotations

import os
import time
from typing import Dict, List, Optional

import torch

from . import native as rt


class ExpertStreamer:
    def __init__(self, model, slots_per_layer: int, policy: str = "impact_weighted_lru", waterline: int = 4, prefetch: bool = False,
                 fetch_deadline_ms: Optional[float] = None, numa_node: int = -1, place_freq: Optional[str] = None,
                 cfg=None, device=None, live_source=None, cpu_offload: Optional[bool] = None, cpu_threads: int = 0):
        """Takes a fully resident ``DeviceModel`` (every MoE layer's arena holds all of this rank's experts), moves
        the slot images to pinned host memory and shrinks every arena to ``slots_per_layer`` slots.
        With ``model = None`` (and ``cfg`` / ``device`` given) the streamer starts empty: pass :meth:`add_layer` as the ``layer_hook`` of
        ``DeviceModel.from_state_dict`` / ``random_init`` so that every MoE layer is moved out as soon as it is built - the model then
        never has to fit in HBM as a whole, only its resident part plus one layer's experts - and call :meth:`attach` at the end."""
        self.model = model
        self.cfg = cfg if cfg is not None else model.cfg
        self.dev = torch.device(device) if device is not None else model.device
        self.slots = slots_per_layer
        self.policy, self.numa_node = policy, numa_node
        self.copy_stream = torch.cuda.Stream(device=self.dev)
        self.te = rt.TransferEngine(n_gpus=1, levels=3, waterline=waterline)
        self.layers: Dict[int, dict] = {}
        self.prefetch = prefetch
        self.trace = open(os.environ["LS_ROUTING_TRACE"], "w") if os.environ.get("LS_ROUTING_TRACE") else None
        self.trace_step = 0
        # LS_FETCH_TRACE: one line per batch of host->device copies (copies, bytes, device time between events on the copy stream):
        # the input of the copy cost-model fit (utils/loader_xray.py fit-constants)
        self.fetch_trace_path = os.environ.get("LS_FETCH_TRACE") or None
        self._fetch_spans: List[tuple] = []
        self._span_start = None
        self.weighted = False                                    # True once configure_eviction() has installed the weighted score
        self.stats = {"hits": 0, "misses": 0, "waves": 0, "bytes_h2d": 0, "degraded_steps": 0, "late_experts": 0, "host_waits": 0}
        self._issued: List[tuple] = []
        self.fetch_deadline_ms = fetch_deadline_ms
        self._copy_done = lambda ev: ev.query()                  # tests replace this to stall a completion on the host side
        self._late: List[tuple] = []                              # copies that missed a deadline: (event, token, layer, expert, slot)
        self._slot_free_ev = None                                 # compute-stream event after the last expert kernels that read the slots
        self.h_ids = None
        self._last_layer = -1
        # GGUF checkpoints: slot images of covered layers come straight from the file into the pinned store (runtime/live_gguf.py);
        # the model builder then leaves those layers' arenas to this streamer (``DeviceModel.from_state_dict(skip_experts=...)``)
        self.live_source = live_source
        # CPU offload of missed experts (opt-in, LSB_STREAM_CPU_OFFLOAD=1): a decode step's experts that are not resident are split
        # between the copy engine and the host's expert kernels (csrc/runtime/cpu_experts.cpp reads the same slot images from the
        # pinned store) so that both finish at about the same time; the CPU never takes work it would finish later than the copy
        if cpu_offload is None:
            cpu_offload = os.environ.get("LSB_STREAM_CPU_OFFLOAD", "0") not in ("", "0")
        self.cpu = rt.CpuExperts(cpu_threads) if cpu_offload else None
        self.cpu_max_rows = 4
        self._cpu_pool = None
        self._cpu_ms = None                                       # measured host time of one expert for one row
        self._cpu_future = None
        self.h_x = None
        self.cpu_partial = None                                   # device fp32 [rows, hidden] to add after the combine (set by run_layer)
        self.stats.update({"cpu_experts": 0, "cpu_wait_ms": 0.0})
        self._place_freq = place_freq or os.environ.get("LS_ARENA_PLACE_FREQ") or None
        if model is not None:
            for i, L in enumerate(model.layers):
                self.add_layer(i, L)
            self.attach(model)

    def add_layer(self, i: int, L: dict):
        """Move the experts of layer ``i`` (``L``: its entry of ``DeviceModel.layers``, arena fully resident) to pinned host memory and
        replace the arena by one of ``slots_per_layer`` slots.  No-op for layers without experts."""
        from ..models.device_model import ExpertArena
        if L.get("arena") is None and self.live_source is not None and self.covers(i):
            return self._add_layer_live(i, L)
        if "arena" not in L or L["arena"] is None:
            return
        cfg = self.cfg
        E_total = cfg.n_routed + cfg.n_shared
        old: ExpertArena = L["arena"]
        so = old.slot_of.cpu().tolist()
        mine = [e for e in range(E_total) if so[e] >= 0]
        # backing store: the native host arena (NUMA-bound slab, page-locked with cudaHostRegister); plain pinned memory if the
        # slab cannot be mapped or registered
        harena = None
        try:
            harena = rt.HostArena(old.ef.stride, len(mine), numa_node=self.numa_node)
            if not harena.pin():
                harena = None
        except (MemoryError, OSError):
            harena = None
        host = harena.tensor() if harena is not None else torch.empty(len(mine), old.ef.stride, dtype=torch.uint8).pin_memory()
        host_row = {}
        for r, e in enumerate(mine):
            if harena is not None:
                slot_h, _ = harena.begin_load(i, e)
                host[slot_h].copy_(old.data[so[e]])
                harena.finish_load(slot_h, True)
                host_row[e] = slot_h
            else:
                host[r].copy_(old.data[so[e]])
                host_row[e] = r
        n = min(self.slots, len(mine))
        assert n >= min(len(mine), cfg.top_k + cfg.n_shared), "the layer needs room for one token's experts"
        new = ExpertArena(old.ef, n, E_total, self.dev)
        L["arena"] = new
        self.layers[i] = {"host": host, "host_row": host_row, "host_arena": harena, "cache": rt.ExpertCache(0, n, self.policy), "arena": new,
                          "expert_stats": rt.ExpertStats(E_total),
                          "slot_of_host": torch.full((E_total,), -1, dtype=torch.int32).pin_memory(),
                          "present": torch.zeros(E_total, dtype=torch.int32, device=self.dev), "mine": set(mine), "pending": {}}
        del old
        if self.model is None:
            torch.cuda.synchronize(self.dev)                     # layer-by-layer loading: give the full arena back before the next layer is built
            torch.cuda.empty_cache()

    def covers(self, i: int) -> bool:
        """Whether layer ``i``'s experts can come straight from the checkpoint file (the model builder may skip its arena)."""
        return self.live_source is not None and self.cfg.is_moe_layer(i) and self.live_source.layout(i) is not None

    def _add_layer_live(self, i: int, L: dict):
        """A covered layer: the host store is filled from the GGUF file, the device arena starts empty with ``slots`` slots."""
        from ..models.device_model import ExpertArena
        cfg = self.cfg
        E_total = cfg.n_routed + cfg.n_shared
        ef = self.live_source.layout(i)
        mine = list(range(E_total))
        harena = None
        try:
            harena = rt.HostArena(ef.stride, len(mine), numa_node=self.numa_node)
            if not harena.pin():
                harena = None
        except (MemoryError, OSError):
            harena = None
        host = harena.tensor() if harena is not None else torch.empty(len(mine), ef.stride, dtype=torch.uint8).pin_memory()
        host_row = {}
        if harena is not None:
            for e in mine:
                host_row[e] = harena.begin_load(i, e)[0]
        else:
            host_row = {e: e for e in mine}
        self.live_source.build_layer(i, mine, host, [host_row[e] for e in mine])
        if harena is not None:
            for e in mine:
                harena.finish_load(host_row[e], True)
        n = min(self.slots, len(mine))
        assert n >= min(len(mine), cfg.top_k + cfg.n_shared), "the layer needs room for one token's experts"
        new = ExpertArena(ef, n, E_total, self.dev)
        L["arena"] = new
        self.layers[i] = {"host": host, "host_row": host_row, "host_arena": harena, "cache": rt.ExpertCache(0, n, self.policy), "arena": new,
                          "expert_stats": rt.ExpertStats(E_total),
                          "slot_of_host": torch.full((E_total,), -1, dtype=torch.int32).pin_memory(),
                          "present": torch.zeros(E_total, dtype=torch.int32, device=self.dev), "mine": set(mine), "pending": {}}

    def attach(self, model):
        """The model's MoE layers are all in: make this streamer the one its steps go through (and pre-warm from the configured
        demand-fetch table)."""
        self.model = model
        torch.cuda.synchronize(self.dev)
        torch.cuda.empty_cache()
        self._last_layer = max(self.layers) if self.layers else -1
        model.streamer = self
        if self._place_freq:
            from ..utils.loader_xray import read_freq_table
            self.prewarm(read_freq_table(self._place_freq))
        return self

    def prewarm(self, freq: Dict[tuple, int]) -> int:
        """Start with the most often FETCHED experts of every layer resident (``freq``: {(layer, expert): demand fetches}, the table
        ``utils/loader_xray.py freq-table`` derives from a recorded run).  Returns the number of experts loaded."""
        n_loaded = 0
        for li, st in self.layers.items():
            ranked = sorted((e for (l, e) in freq if l == li and e in st["mine"]), key=lambda e: -freq[(li, e)])
            for e in ranked[: st["arena"].n_slots]:
                if st["cache"].lookup(li, e) < 0 and self._reserve(li, st, e):
                    n_loaded += 1
            self._issue()
            self._settle()
        torch.cuda.synchronize(self.dev)
        return n_loaded

    # ------------------------------------------------------------------ residency
    def _reserve(self, li: int, st: dict, e: int, priority: int = 0) -> bool:
        """Reserve a slot for expert ``e`` of layer ``li`` (evicting the best unlocked ready victim when the layer is
        full) and queue its host->device copy.  False = every slot is locked or still loading."""
        cache: rt.ExpertCache = st["cache"]
        try:
            slot = cache.reserve(li, e, rt.ZONE_STREAMING, True)
        except rt.NativeError:
            victim = cache.pick_victim(-1)
            if victim is None:
                return False
            cache.evict(victim[1], victim[2])
            st["slot_of_host"][victim[2]] = -1
            slot = cache.reserve(li, e, rt.ZONE_STREAMING, True)
        tok = self.te.submit(li, e, 0, rt.TransferEngine.H2D, priority, st["arena"].ef.stride)
        st["pending"][tok] = (e, slot)
        return True

    def _issue(self):
        """Start every copy the transfer engine releases (priority order, bounded in-flight count) on the side stream."""
        now = time.monotonic_ns()
        while True:
            tok = self.te.next_to_issue(0, now)
            if not tok:
                if self.te.queued(0) and self.te.in_flight(0):
                    before = self.te.in_flight(0)
                    self._settle()                               # waterline reached: gate what is out, then continue issuing
                    if self.te.in_flight(0) < before:
                        continue
                break                                            # nothing more to issue (or only stalled copies are in flight)
            info = self.te.info(tok)
            lst = self.layers[info["layer"]]
            e, slot = lst["pending"][tok]
            with torch.cuda.stream(self.copy_stream):
                if self._slot_free_ev is not None:
                    self.copy_stream.wait_event(self._slot_free_ev)  # the kernels that last read this layer's slots have finished (device side)
                if self.fetch_trace_path and self._span_start is None:
                    self._span_start = torch.cuda.Event(enable_timing=True)
                    self._span_start.record(self.copy_stream)
                lst["arena"].data[slot].copy_(lst["host"][lst["host_row"][e]], non_blocking=True)
            self.stats["bytes_h2d"] += lst["arena"].ef.stride
            self._issued.append((tok, info["layer"], e, slot))

    def _mark_landed(self, tok, li, e, slot, now):
        lst = self.layers[li]
        self.te.complete(tok, now)
        lst["pending"].pop(tok, None)
        lst["cache"].mark_ready(li, e)
        lst["slot_of_host"][e] = slot

    def _settle(self) -> List[tuple]:
        """Gate the issued copies on the device and publish their slots.  Without a deadline the compute stream is made to wait
        for the copies' event and the host goes on at once.  With ``fetch_deadline_ms`` the host polls the event up to the
        deadline; copies that have not landed are returned as late [(layer, expert)] - their slots stay reserved, they are
        published by a later call, and the caller runs this step without them."""
        self._retire_late()
        if not self._issued:
            return []
        ev = torch.cuda.Event(enable_timing=bool(self.fetch_trace_path))
        ev.record(self.copy_stream)
        if self._span_start is not None:
            self._fetch_spans.append((self.trace_step, len(self._issued), sum(self.layers[li]["arena"].ef.stride for _, li, _, _ in self._issued),
                                      self._span_start, ev))
            self._span_start = None
        late: List[tuple] = []
        now = time.monotonic_ns()
        if self.fetch_deadline_ms is not None:
            t_end = time.monotonic() + self.fetch_deadline_ms / 1e3
            done = self._copy_done(ev)
            while not done and time.monotonic() < t_end:
                time.sleep(20e-6)
                done = self._copy_done(ev)
            self.stats["host_waits"] += 1
            if not done:
                for tok, li, e, slot in self._issued:
                    self._late.append((ev, tok, li, e, slot))
                    late.append((li, e))
                self.stats["late_experts"] += len(late)
                self._issued = []
                return late
        torch.cuda.current_stream(self.dev).wait_event(ev)       # device-side gate: kernels launched from here on see the copies
        for tok, li, e, slot in self._issued:
            self._mark_landed(tok, li, e, slot, now)
        self._issued = []
        self.te.poll()
        return late

    def _retire_late(self):
        """Copies that missed an earlier deadline and have landed since become ready now (the retry half of deadline -> degraded -> retry)."""
        if not self._late:
            return
        keep = []
        now = time.monotonic_ns()
        for ev, tok, li, e, slot in self._late:
            if self._copy_done(ev):
                torch.cuda.current_stream(self.dev).wait_event(ev)
                self._mark_landed(tok, li, e, slot, now)
            else:
                keep.append((ev, tok, li, e, slot))
        self._late = keep

    # ------------------------------------------------------------------ per-layer driver
    def run_layer(self, model, li: int, arena, ws, R: int):
        """Expert kernels of one MoE layer under the capped cache.  Returns the table the combine uses to tell which
        experts' outputs exist (0 for this rank's experts that were computed, -1 otherwise)."""
        st = self.layers[li]
        cache: rt.ExpertCache = st["cache"]
        # the one host wait of the layer: which experts does the step need?  (ids | weights through one pinned buffer)
        n_pairs = R * ws.S
        if self.h_ids is None or self.h_ids.numel() < 2 * n_pairs:
            self.h_ids = torch.zeros(2 * max(n_pairs, 64), dtype=torch.int32).pin_memory()
        cur = torch.cuda.current_stream(self.dev)
        self.h_ids[:n_pairs].copy_(ws.ids[:R].reshape(-1), non_blocking=True)
        self.h_ids[n_pairs: 2 * n_pairs].copy_(ws.wts[:R].reshape(-1).view(torch.int32), non_blocking=True)
        self.cpu_partial = None
        use_cpu = self.cpu is not None and R <= self.cpu_max_rows and st["arena"].ef.fmt <= 3 and not st["arena"].ef.fmt_down1
        if use_cpu:
            if self.h_x is None:
                self.h_x = torch.zeros(self.cpu_max_rows, self.cfg.hidden, dtype=torch.bfloat16).pin_memory()
                self.d_ycpu = torch.zeros(self.cpu_max_rows, self.cfg.hidden, device=self.dev)
                self.h_ycpu = torch.zeros(self.cpu_max_rows, self.cfg.hidden).pin_memory()
            self.h_x[:R].copy_(ws.x[:R], non_blocking=True)          # the layer's normalised input rows ride along with the routing
        ev_ids = torch.cuda.Event()
        ev_ids.record(cur)
        ev_ids.synchronize()
        ids = self.h_ids[:n_pairs]
        wts = self.h_ids[n_pairs: 2 * n_pairs].view(torch.float32)
        need: Dict[int, float] = {}
        for e, w in zip(ids.tolist(), wts.tolist()):
            if e in st["mine"]:
                need[e] = need.get(e, 0.0) + w
        todo = sorted(need, key=lambda e: -need[e])              # heaviest experts first
        if self.trace is not None:                               # LS_ROUTING_TRACE: input of the offline cache replay (utils/cache_sim.py)
            self.trace.write(f"{self.trace_step} {li} {' '.join(str(e) for e in todo)}\n")
        if li == self._last_layer:
            self.trace_step += 1                                 # counts steps for both traces (routing, copies)
        st["expert_stats"].observe(todo, [need[e] for e in todo])
        if use_cpu:
            todo = self._offload_to_cpu(li, st, ws, R, todo, ids, wts)
        model._moe_prepare(arena, ws, R)
        st["present"].fill_(-1)
        degraded = False
        while todo:
            wave: List[int] = []
            fetched: List[int] = []
            locked = set()
            late_pre = set()

            def lock_landed():
                # a copy that has landed is evictable until it is locked: pin this wave's experts as soon as they are ready
                for f in fetched:
                    if f not in locked and cache.is_ready(li, f):
                        cache.lock(li, f)
                        locked.add(f)

            for e in todo:
                if len(wave) == arena.n_slots:
                    break
                if cache.lookup(li, e) >= 0 and not cache.is_ready(li, e):
                    self._issue()                                # a prefetch of this expert is still on its way
                    self._settle()
                    lock_landed()
                    if not cache.is_ready(li, e):                # ... and missed the deadline: this step goes on without it
                        late_pre.add(e)
                        continue
                if cache.lookup(li, e) >= 0:
                    self.stats["hits"] += 1
                    cache.lock(li, e)
                    locked.add(e)
                elif self._reserve(li, st, e):
                    self.stats["misses"] += 1
                    fetched.append(e)
                else:
                    break                                        # nothing evictable any more: run what is resident
                wave.append(e)
            if not wave and not late_pre:
                raise RuntimeError(f"layer {li}: no expert slot can be freed")
            self._issue()
            self._settle()
            lock_landed()
            # with a fetch deadline some of the wave's copies may not have landed (stalled, or still queued behind stalled ones):
            # this step runs without those experts (degraded); their copies keep going and are published by a later call
            late = {e for e in wave if not cache.is_ready(li, e)} | late_pre
            if late:
                degraded = True
                wave = [e for e in wave if e not in late]
            so = torch.full_like(st["slot_of_host"], -1)
            for e in wave:
                cache.touch(li, e, need[e])
                so[e] = st["slot_of_host"][e]
            arena.slot_of.copy_(so, non_blocking=True)           # only this wave's experts are visible to the kernels
            if wave:
                model._moe_experts(arena, ws, R, None)
                st["present"][torch.tensor(wave, dtype=torch.long, device=self.dev)] = 0
            # slots may be reused by the next wave / layer: the side stream waits for these kernels on the device, the host does not
            self._slot_free_ev = torch.cuda.Event()
            self._slot_free_ev.record(torch.cuda.current_stream(self.dev))
            for e in wave:
                cache.unlock(li, e)
            done = set(wave) | late
            todo = [e for e in todo if e not in done]
            self.stats["waves"] += 1
        if self._cpu_future is not None:
            # the host's share: wait for it (it was sized to finish with the copies), ship [rows, hidden] fp32 and let the caller add it
            t0 = time.perf_counter()
            y = self._cpu_future.result()
            self.stats["cpu_wait_ms"] += (time.perf_counter() - t0) * 1e3
            self._cpu_future = None
            self.h_ycpu[:R].copy_(y)
            self.d_ycpu[:R].copy_(self.h_ycpu[:R], non_blocking=True)
            self.stats["bytes_h2d"] += R * self.cfg.hidden * 4
            self.cpu_partial = self.d_ycpu[:R]
        if degraded:
            self.stats["degraded_steps"] += 1
        if self.weighted:
            cache.end_step()                                     # fold this pass's touches into frequency / autocorrelation / hysteresis
        if self.prefetch:
            self._prefetch_next(model, li, ws, R, list(need))
        return st["present"]

    def _offload_to_cpu(self, li: int, st: dict, ws, R: int, todo: List[int], ids, wts) -> List[int]:
        """Split the step's missed experts between the copy engine and the host kernels; returns the experts left for the GPU.
        With m missed experts, a copy costing f and a host expert costing c, n = m f / (c + f) of them go to the host: both sides
        then finish together, and the host is never given an expert it would finish after the copy it replaces."""
        import ctypes
        from concurrent.futures import ThreadPoolExecutor
        cache = st["cache"]
        miss = [e for e in todo if cache.lookup(li, e) < 0]
        if not miss:
            return todo
        ef = st["arena"].ef
        if self._cpu_pool is None:
            self._cpu_pool = ThreadPoolExecutor(max_workers=1)
        if self._cpu_ms is None:                                    # one timed expert on the host, once
            x0 = torch.zeros(1, self.cfg.hidden)
            e0 = miss[0]
            t0 = time.perf_counter()
            self.cpu.ffn(ctypes.addressof(ef), st["host"][st["host_row"][e0]], x0, self.cfg.swiglu_limit)
            self.cpu.ffn(ctypes.addressof(ef), st["host"][st["host_row"][e0]], x0, self.cfg.swiglu_limit)
            self._cpu_ms = max(1e-3, (time.perf_counter() - t0) * 1e3 / 2)
        gbs = self.te.bandwidth_gbs(0, 0) or 50.0
        f_ms = ef.stride / (max(gbs, 1.0) * 1e6)
        c_ms = self._cpu_ms * R
        m = len(miss)
        lo = min(m, int(m * f_ms / (c_ms + f_ms)))
        n_cpu = min((lo, min(m, lo + 1)), key=lambda n: max(n * c_ms, (m - n) * f_ms))      # both sides finish together, whichever split is faster
        if n_cpu <= 0:
            return todo
        mine = set(miss[-n_cpu:])                                   # the lightest missed experts: the heavier ones are worth caching
        n_pairs = R * ws.S
        ids_cpu = torch.where(torch.isin(ids, torch.tensor(sorted(mine), dtype=ids.dtype)), ids, torch.full_like(ids, -1)).view(R, ws.S).clone()
        wts_cpu = wts.view(R, ws.S).clone()
        x = self.h_x[:R].float()
        slots = {e: st["host"][st["host_row"][e]] for e in mine}
        E_total = self.cfg.n_routed + self.cfg.n_shared
        self._cpu_future = self._cpu_pool.submit(self.cpu.moe_layer, ctypes.addressof(ef), slots, E_total, x, ids_cpu, wts_cpu, self.cfg.swiglu_limit)
        self.stats["cpu_experts"] += n_cpu
        return [e for e in todo if e not in mine]

    def _prescope(self, model, nxt: int, ws, R: int) -> List[int]:
        """Pre-gating ("prescope"): run the NEXT MoE layer's router on this layer's input.  The residual stream changes
        slowly from layer to layer, so the experts it picks predict the real routing well; the prediction only steers
        prefetch, never the computation."""
        cfg = model.cfg
        L = model.layers[nxt]
        if not hasattr(ws, "_pre"):
            dev = model.device
            ws._pre = (torch.zeros(ws.R, cfg.n_routed, device=dev), torch.zeros(ws.R, ws.S, dtype=torch.int32, device=dev), torch.zeros(ws.R, ws.S, device=dev))
        lg, ids, wts = ws._pre
        from ..ops import _native as nat
        L["router"](lg, ws.x, R)
        sc = {"sigmoid": 0, "softmax": 1, "sqrtsoftplus": 2}[cfg.scoring]
        nat.call("lsb_router_topk", lg, L["router_bias"], ids, wts, R, cfg.n_routed, cfg.top_k, cfg.n_group, cfg.topk_group, sc,
                 int(cfg.norm_topk_prob), cfg.routed_scale, cfg.n_shared, cfg.n_routed)
        flat = ids[:R].reshape(-1).cpu().tolist()
        seen, out = set(), []
        for e in flat:
            if e >= 0 and e not in seen:
                seen.add(e)
                out.append(e)
        return out

    def _prefetch_next(self, model, li: int, ws, R: int, fallback: List[int]):
        """Request the experts the next MoE layer will probably route to, at the lowest priority, so their copies overlap
        this layer's combine and the next layer's attention."""
        nxt = min((j for j in self.layers if j > li), default=None)
        if nxt is None:
            return
        st = self.layers[nxt]
        experts = self._prescope(model, nxt, ws, R) if R <= 4 else fallback
        self.stats["prefetch_requests"] = self.stats.get("prefetch_requests", 0) + len(experts)
        for e in experts[: max(0, st["arena"].n_slots // 2)]:
            if e in st["mine"] and st["cache"].lookup(nxt, e) < 0:
                if not self._reserve(nxt, st, e, priority=2):
                    break
        self._issue()                                            # copies overlap the rest of this layer and the next attention

    def configure_eviction(self, section: dict):
        """Switch every layer's cache to the weighted eviction score of the ``memory.expert_cache`` configuration section (policy + the
        seven weights).  May be called again at any time: the fields are live-changeable."""
        self.weighted = True
        for st in self.layers.values():
            st["cache"].configure(section)

    def flush_fetch_trace(self) -> int:
        """Write the copy batches recorded so far to ``LS_FETCH_TRACE`` (appending) and forget them; returns how many."""
        if not self.fetch_trace_path or not self._fetch_spans:
            return 0
        torch.cuda.synchronize(self.dev)
        with open(self.fetch_trace_path, "a") as fh:
            if fh.tell() == 0:
                fh.write("# W step copies bytes device_us\n")
            for step, n, nbytes, e0, e1 in self._fetch_spans:
                fh.write(f"W {step} {n} {nbytes} {e0.elapsed_time(e1) * 1e3:.1f}\n")
        n = len(self._fetch_spans)
        self._fetch_spans = []
        return n

    def summary(self) -> dict:
        self.flush_fetch_trace()
        tot = max(1, self.stats["hits"] + self.stats["misses"])
        return dict(self.stats, hit_rate=self.stats["hits"] / tot, h2d_gbs=self.te.bandwidth_gbs(0, 0),
                    numa_bound_layers=sum(1 for st in self.layers.values() if st["host_arena"] is not None and st["host_arena"].numa_bound))

    def expert_frequencies(self, li: int):
        """Decayed per-expert selection frequency of one layer (native ``ExpertStats``, fed by every step's routing)."""
        return self.layers[li]["expert_stats"].frequencies()
