"""Capped VRAM expert cache backed by pinned host memory (expert streaming).

Each MoE layer keeps ``slots_per_layer`` expert slots in HBM; every expert's slot image lives in a
pinned host store.  Per layer and step:
  1. the routed expert ids come back to the host (one small D2H copy, the only host round trip),
  2. missing experts are fetched host->device with pinned ``cudaMemcpyAsync`` on a side stream -
     what is fetched when is decided by the native ``TransferEngine`` (de-duplication, priorities,
     in-flight waterline) and where it lands by the native ``ExpertCache`` (impact-weighted LRU,
     locked while in use),
  3. the compute stream waits on the copies' event and runs the expert kernels over the resident
     experts; when a step needs more experts than the layer has slots (prefill chunks) this repeats
     in waves, and the combine runs once at the end.
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
    def __init__(self, model, slots_per_layer: int, policy: str = "impact_weighted_lru", waterline: int = 4, prefetch: bool = False):
        """Takes a fully resident ``DeviceModel`` (every MoE layer's arena holds all of this rank's experts), moves
        the slot images to pinned host memory and shrinks every arena to ``slots_per_layer`` slots."""
        from ..models.device_model import ExpertArena
        self.model, self.dev = model, model.device
        self.slots = slots_per_layer
        self.copy_stream = torch.cuda.Stream(device=self.dev)
        self.te = rt.TransferEngine(n_gpus=1, levels=3, waterline=waterline)
        self.layers: Dict[int, dict] = {}
        self.prefetch = prefetch
        self.trace = open(os.environ["LS_ROUTING_TRACE"], "w") if os.environ.get("LS_ROUTING_TRACE") else None
        self.trace_step = 0
        self.weighted = False                                    # True once configure_eviction() has installed the weighted score
        self.stats = {"hits": 0, "misses": 0, "waves": 0, "bytes_h2d": 0}
        self._issued: List[tuple] = []
        cfg = model.cfg
        E_total = cfg.n_routed + cfg.n_shared
        for i, L in enumerate(model.layers):
            if "arena" not in L:
                continue
            old: ExpertArena = L["arena"]
            so = old.slot_of.cpu().tolist()
            mine = [e for e in range(E_total) if so[e] >= 0]
            host = torch.empty(len(mine), old.ef.stride, dtype=torch.uint8).pin_memory()
            host_row = {}
            for r, e in enumerate(mine):
                host[r].copy_(old.data[so[e]])
                host_row[e] = r
            n = min(slots_per_layer, len(mine))
            assert n >= min(len(mine), cfg.top_k + cfg.n_shared), "the layer needs room for one token's experts"
            new = ExpertArena(old.ef, n, E_total, self.dev)
            L["arena"] = new
            self.layers[i] = {"host": host, "host_row": host_row, "cache": rt.ExpertCache(0, n, policy), "arena": new,
                              "slot_of_host": torch.full((E_total,), -1, dtype=torch.int32).pin_memory(),
                              "present": torch.zeros(E_total, dtype=torch.int32, device=self.dev), "mine": set(mine), "pending": {}}
            del old
        torch.cuda.synchronize(self.dev)
        torch.cuda.empty_cache()
        self._last_layer = max(self.layers) if self.layers else -1
        model.streamer = self

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
                    self._settle()                               # waterline reached: drain, then continue issuing
                    continue
                break
            info = self.te.info(tok)
            lst = self.layers[info["layer"]]
            e, slot = lst["pending"][tok]
            with torch.cuda.stream(self.copy_stream):
                lst["arena"].data[slot].copy_(lst["host"][lst["host_row"][e]], non_blocking=True)
            self.stats["bytes_h2d"] += lst["arena"].ef.stride
            self._issued.append((tok, info["layer"], e, slot))

    def _settle(self):
        """Wait for the side stream; every issued copy has landed: mark it ready and publish its slot."""
        if not self._issued:
            return
        self.copy_stream.synchronize()
        now = time.monotonic_ns()
        for tok, li, e, slot in self._issued:
            lst = self.layers[li]
            self.te.complete(tok, now)
            lst["pending"].pop(tok, None)
            lst["cache"].mark_ready(li, e)
            lst["slot_of_host"][e] = slot
        self._issued = []
        self.te.poll()

    # ------------------------------------------------------------------ per-layer driver
    def run_layer(self, model, li: int, arena, ws, R: int):
        """Expert kernels of one MoE layer under the capped cache.  Returns the table the combine uses to tell which
        experts' outputs exist (0 for this rank's experts that were computed, -1 otherwise)."""
        st = self.layers[li]
        cache: rt.ExpertCache = st["cache"]
        ids = ws.ids[:R].reshape(-1).cpu()                       # the one host round trip: which experts does the step need?
        wts = ws.wts[:R].reshape(-1).cpu()
        need: Dict[int, float] = {}
        for e, w in zip(ids.tolist(), wts.tolist()):
            if e in st["mine"]:
                need[e] = need.get(e, 0.0) + w
        todo = sorted(need, key=lambda e: -need[e])              # heaviest experts first
        if self.trace is not None:                               # LS_ROUTING_TRACE: input of the offline cache replay (utils/cache_sim.py)
            self.trace.write(f"{self.trace_step} {li} {' '.join(str(e) for e in todo)}\n")
            if li == self._last_layer:
                self.trace_step += 1
        model._moe_prepare(arena, ws, R)
        st["present"].fill_(-1)
        while todo:
            wave: List[int] = []
            fetched: List[int] = []
            locked = set()

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
            if not wave:
                raise RuntimeError(f"layer {li}: no expert slot can be freed")
            self._issue()
            self._settle()
            lock_landed()
            so = torch.full_like(st["slot_of_host"], -1)
            for e in wave:
                cache.touch(li, e, need[e])
                so[e] = st["slot_of_host"][e]
            arena.slot_of.copy_(so)                              # only this wave's experts are visible to the kernels
            model._moe_experts(arena, ws, R, None)
            st["present"][torch.tensor(wave, dtype=torch.long, device=self.dev)] = 0
            torch.cuda.current_stream(self.dev).synchronize()    # slots may be reused by the next wave / layer
            for e in wave:
                cache.unlock(li, e)
            done = set(wave)
            todo = [e for e in todo if e not in done]
            self.stats["waves"] += 1
        if self.weighted:
            cache.end_step()                                     # fold this pass's touches into frequency / autocorrelation / hysteresis
        if self.prefetch:
            self._prefetch_next(model, li, ws, R, list(need))
        return st["present"]

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

    def summary(self) -> dict:
        tot = max(1, self.stats["hits"] + self.stats["misses"])
        return dict(self.stats, hit_rate=self.stats["hits"] / tot, h2d_gbs=self.te.bandwidth_gbs(0, 0))
