"""Prefix cache: a radix tree of frozen holder sequences.

A finished prompt leaves a *holder* (a forked, never-appending sequence) registered at
grid-aligned lengths; a new request whose prompt shares a prefix forks from the deepest holder
instead of prefilling those tokens again (copy-on-write pages).  Nodes exist only at multiples
of ``grid`` tokens (or the exact prompt body), so cache ON and OFF run the same chunk shapes and
give identical tokens.  Eviction is leaf-only, least-recently-used first, deepest first among
equals; the token budget counts unique (edge) tokens.  Models with recurrent state (KDA) can only
be forked at a holder's exact frontier.
Tiering of idle holders (``idle_sweep``, called by the serving loop when it has nothing to do, never on the request path):
first hop - a holder nobody hit for ``hibernate_idle_seconds`` moves its KV pages to pinned host memory (``Engine.hibernate``) and
gives its HBM pages back; second hop - a hibernated LEAF holder idle for ``spill.idle_seconds`` is written to a file under
``spill.path`` (``Engine.spill``), least recently used first, at most one per sweep, under a byte cap that is enforced BEFORE the
write (over the cap: the least recently used spilled holder is dropped with its file, once).  The directory is a cache, never a
store: its ``ls-spill-*.kvspill`` files are reclaimed at start-up, and a lost or unreadable file degrades to a cache MISS (the
holder is dropped, the request prefills again).  An unwritable directory disables the second hop at boot, loudly.
Reference: PrefixCache in python/orchestrator/orchestrator.py:598-643,804-1272 (radix tree of frozen
holders, touch propagation, leaf-only LRU eviction, fork-with-evict-retry), PrefixSpillConfig :455-484 (cold spill policy).
"""
from __future__ import annotations

import glob
import itertools
import logging
import os
import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

log = logging.getLogger("layerstorm_b200.prefix_cache")


@dataclass
class PrefixSpillConfig:
    enabled: bool = False
    path: str = "~/.layerstorm/prefix-cache"
    max_mib: int = 32768
    idle_seconds: float = 300.0

    @classmethod
    def from_config(cls, cfg: dict) -> "PrefixSpillConfig":
        ps = (cfg or {}).get("_internal-prefix_spill") or {}
        return cls(bool(ps.get("enabled", True)), str(ps.get("path", "~/.layerstorm/prefix-cache")), int(ps.get("max_mib", 32768)),
                   float(ps.get("idle_seconds", 300.0)))


@dataclass
class PrefixCacheConfig:
    enabled: bool = True
    grid: int = 64                    # node granularity in tokens
    max_tokens: int = 1 << 20         # budget over unique cached tokens
    max_holders: int = 64
    min_prefix: int = 64
    hibernate_holders: bool = False   # idle holders move to pinned host memory (needs Engine.enable_kv_tiering)
    hibernate_idle_seconds: float = 30.0
    spill: Optional[PrefixSpillConfig] = None


@dataclass
class _Node:
    depth: int                        # total tokens from the root (a multiple of the grid)
    holder: Optional[int] = None      # engine sequence id holding KV for [0, depth)
    children: Dict[Tuple[int, ...], "_Node"] = field(default_factory=dict)   # keyed by the next grid block
    parent: Optional["_Node"] = None
    key: Tuple[int, ...] = ()
    last_used: int = 0


class PrefixCache:
    def __init__(self, engine, cfg: Optional[PrefixCacheConfig] = None):
        self.engine, self.cfg = engine, cfg or PrefixCacheConfig()
        self.root = _Node(0)
        self.exact: Dict[Tuple[int, ...], Tuple[int, int]] = {}    # recurrent models: full prefix -> (holder, last_used)
        self._clock = itertools.count(1)
        self.hits = self.misses = self.hit_tokens = 0
        self._hit_time: Dict[int, float] = {}                      # holder -> wall-clock time of its last hit / registration
        self._spilled: Dict[int, Tuple[str, int]] = {}             # holder -> (file, bytes)
        self.spill_stats = {"hibernated": 0, "spilled": 0, "spill_bytes": 0, "cap_evictions": 0, "lost_files": 0}
        self.spill_dir: Optional[str] = None
        sp = self.cfg.spill
        if sp is not None and sp.enabled and self.cfg.hibernate_holders:
            d = os.path.expanduser(sp.path)
            try:
                os.makedirs(d, exist_ok=True)
                for f in glob.glob(os.path.join(d, "ls-spill-*.kvspill")):          # a cache, never a store: start empty
                    os.remove(f)
                probe = os.path.join(d, f".probe-{os.getpid()}")
                open(probe, "wb").close()
                os.remove(probe)
                self.spill_dir = d
            except OSError as e:
                log.warning("prefix-cache spill DISABLED: %s is not writable (%s)", d, e)

    @property
    def recurrent(self) -> bool:
        return bool(getattr(self.engine, "has_recurrent_state", False))

    # ---- queries ----
    def _walk(self, tokens: List[int], limit: Optional[int] = None) -> _Node:
        """Deepest node whose path (whole grid blocks) is a prefix of ``tokens[:limit]``."""
        g, node = self.cfg.grid, self.root
        n = len(tokens) if limit is None else limit
        while node.depth + g <= n:
            ch = node.children.get(tuple(tokens[node.depth: node.depth + g]))
            if ch is None:
                break
            node = ch
        return node

    @staticmethod
    def _any_holder(node: _Node) -> Optional[int]:
        stack = [node]
        while stack:
            n = stack.pop()
            if n.holder is not None:
                return n.holder
            stack.extend(n.children.values())
        return None

    def lookup(self, tokens: List[int]) -> Tuple[Optional[int], int]:
        """(holder sequence id, usable prefix length) for the longest cached prefix, or (None, 0).  At
        least one prompt token is always left to prefill so the request gets fresh logits.  The holder
        may be longer than the prefix: forks are truncating."""
        if not self.cfg.enabled:
            return None, 0
        if self.recurrent:
            best = None
            for key, (holder, _) in self.exact.items():
                if len(key) < len(tokens) and (best is None or len(key) > len(best[0])) and tuple(tokens[: len(key)]) == key:
                    best = (key, holder)
            if best is None:
                self.misses += 1
                return None, 0
            self.exact[best[0]] = (best[1], next(self._clock))
            self._hit_time[best[1]] = time.monotonic()
            self.hits += 1
            self.hit_tokens += len(best[0])
            return best[1], len(best[0])
        node = self._walk(tokens, len(tokens) - 1)
        holder = self._any_holder(node) if node.depth >= max(self.cfg.min_prefix, 1) else None
        if holder is None:
            self.misses += 1
            return None, 0
        t = next(self._clock)
        stack = [node]
        while stack:                     # touch the subtree that could serve this prefix and the ancestors
            n = stack.pop()
            n.last_used = t
            stack.extend(n.children.values())
        n = node.parent
        while n is not None:
            n.last_used = t
            n = n.parent
        self.hits += 1
        self.hit_tokens += node.depth
        self._hit_time[holder] = time.monotonic()
        return holder, node.depth

    def _nodes(self):
        stack = [self.root]
        while stack:
            n = stack.pop()
            stack.extend(n.children.values())
            yield n

    def total_tokens(self) -> int:
        if self.recurrent:
            return sum(len(k) for k in self.exact)
        return sum(self.cfg.grid for n in self._nodes() if n is not self.root)

    def holders(self) -> int:
        if self.recurrent:
            return len(self.exact)
        return sum(1 for n in self._nodes() if n.holder is not None)

    # ---- updates ----
    def register(self, seq_id: int, tokens: List[int]) -> Optional[int]:
        """Freeze a copy of ``seq_id`` (whose KV covers ``tokens``) at the largest grid-aligned length
        (recurrent models: at the exact length); returns the holder id or None."""
        if not self.cfg.enabled:
            return None
        if self.recurrent:
            key = tuple(tokens)
            if len(key) < self.cfg.min_prefix:
                return None
            if key in self.exact:
                self.exact[key] = (self.exact[key][0], next(self._clock))
                return self.exact[key][0]
            while self.total_tokens() + len(key) > self.cfg.max_tokens or self.holders() >= self.cfg.max_holders:
                if not self.evict_one():
                    return None
            try:
                h = self.engine.fork_sequence(seq_id, len(key))
            except Exception:  # noqa: BLE001 - caching is best effort
                return None
            self.exact[key] = (h, next(self._clock))
            self._hit_time[h] = time.monotonic()
            return h
        g = self.cfg.grid
        depth = (len(tokens) // g) * g
        if depth < max(self.cfg.min_prefix, g):
            return None
        node = self._walk(tokens, depth)
        if node.depth == depth and node.holder is not None:
            node.last_used = next(self._clock)
            return node.holder
        while self.total_tokens() + (depth - node.depth) > self.cfg.max_tokens or self.holders() >= self.cfg.max_holders:
            if not self.evict_one():
                return None
            node = self._walk(tokens, depth)
        try:
            holder = self.engine.fork_sequence(seq_id, depth)
        except Exception:  # noqa: BLE001
            return None
        t = next(self._clock)
        while node.depth < depth:
            key = tuple(tokens[node.depth: node.depth + g])
            ch = _Node(node.depth + g, parent=node, key=key, last_used=t)
            node.children[key] = ch
            node = ch
        node.holder, node.last_used = holder, t
        self._hit_time[holder] = time.monotonic()
        return holder

    def fork_from(self, tokens: List[int]) -> Tuple[Optional[int], int]:
        """New live sequence sharing the longest cached prefix: (seq id, prefix length)."""
        holder, n = self.lookup(tokens)
        if holder is None:
            return None, 0
        for attempt in range(2):
            try:
                sid = self.engine.fork_sequence(holder, n)
                self._spilled.pop(holder, None)                     # (a spilled holder came back through the engine)
                return sid, n
            except (OSError, ValueError) as e:                     # its spill file is gone or unreadable: a cache miss, never a failure
                log.warning("prefix holder %d lost its spill file (%s): dropped", holder, e)
                self.spill_stats["lost_files"] += 1
                self._drop_holder(holder)
                self.hits -= 1
                self.misses += 1
                return None, 0
            except Exception:  # noqa: BLE001
                if attempt or not self.evict_one(protect=holder):
                    break
        return None, 0

    # ---- tiering of idle holders ----
    def _holder_entries(self):
        """(holder, logical last use, is a leaf) of every holder."""
        if self.recurrent:
            for k, (h, lu) in self.exact.items():
                yield h, lu, True
            return
        for n in self._nodes():
            if n.holder is not None:
                yield n.holder, n.last_used, not n.children

    def _drop_holder(self, holder: int):
        self._spilled.pop(holder, None)
        self._hit_time.pop(holder, None)
        if self.recurrent:
            for k, (h, _) in list(self.exact.items()):
                if h == holder:
                    del self.exact[k]
        else:
            for n in self._nodes():
                if n.holder == holder:
                    n.holder = None
                    while n is not self.root and not n.children and n.holder is None:
                        del n.parent.children[n.key]
                        n = n.parent
                    break
        try:
            self.engine.free_sequence(holder)
        except Exception:  # noqa: BLE001 - the engine may already have dropped it
            pass

    def idle_sweep(self, now: Optional[float] = None) -> dict:
        """One pass of the idle-time tiering policy (see the module text).  Returns what it did."""
        eng = self.engine
        did = {"hibernated": 0, "spilled": 0}
        if not (self.cfg.enabled and self.cfg.hibernate_holders) or not hasattr(eng, "hibernated"):
            return did
        now = time.monotonic() if now is None else now
        entries = sorted(self._holder_entries(), key=lambda t: t[1])
        spilled_in_engine = getattr(eng, "spilled", {})
        for h, _, _ in entries:                                     # first hop: idle holders leave HBM
            if h in eng.hibernated or h in spilled_in_engine:
                continue
            if now - self._hit_time.get(h, now) >= self.cfg.hibernate_idle_seconds:
                try:
                    eng.hibernate(h)
                    did["hibernated"] += 1
                    self.spill_stats["hibernated"] += 1
                except (RuntimeError, NotImplementedError):         # cold pool full / not available: stays hot
                    break
        sp = self.cfg.spill
        if self.spill_dir is None or sp is None:
            return did
        cap = sp.max_mib << 20
        for h, _, leaf in entries:                                  # second hop: at most one hibernated leaf per sweep, LRU first
            if not leaf or h not in eng.hibernated or now - self._hit_time.get(h, now) < sp.idle_seconds:
                continue
            per_page = sum(t[0].numel() * t.element_size() for t in list(eng.cold_kv.values()) + list(eng.cold_idx.values()))
            need = len(eng.hibernated[h]) * per_page
            used = sum(b for _, b in self._spilled.values())
            if used + need > cap:                                   # the cap is enforced before the write: drop the LRU spilled holder, once
                victims = [x for x, _, _ in entries if x in self._spilled and x != h]
                if not victims or need > cap:
                    break
                self._drop_holder(victims[0])
                self.spill_stats["cap_evictions"] += 1
                used = sum(b for _, b in self._spilled.values())
                if used + need > cap:
                    break
            path = os.path.join(self.spill_dir, f"ls-spill-{os.getpid()}-{h}-{next(self._clock)}.kvspill")
            try:
                nbytes = eng.spill(h, path)
            except OSError as e:
                log.warning("prefix-cache spill failed (%s): second hop disabled", e)
                self.spill_dir = None
                break
            self._spilled[h] = (path, nbytes)
            did["spilled"] += 1
            self.spill_stats["spilled"] += 1
            self.spill_stats["spill_bytes"] += nbytes
            break
        return did

    def evict_one(self, protect: Optional[int] = None) -> bool:
        """Drop the least recently used leaf holder (deepest first among equals)."""
        if self.recurrent:
            cands = [(lu, -len(k), k) for k, (h, lu) in self.exact.items() if h != protect]
            if not cands:
                return False
            k = min(cands)[2]
            h = self.exact.pop(k)[0]
            self._spilled.pop(h, None)
            self._hit_time.pop(h, None)
            self.engine.free_sequence(h)
            return True
        best = None
        for n in self._nodes():
            if n is self.root or n.children or n.holder is None or n.holder == protect:
                continue
            if best is None or (n.last_used, -n.depth) < (best.last_used, -best.depth):
                best = n
        if best is None:
            return False
        self._spilled.pop(best.holder, None)
        self._hit_time.pop(best.holder, None)
        self.engine.free_sequence(best.holder)
        best.holder = None
        n = best
        while n is not self.root and not n.children and n.holder is None:   # prune empty leaves
            del n.parent.children[n.key]
            n = n.parent
        return True

    def clear(self):
        while self.evict_one():
            pass
