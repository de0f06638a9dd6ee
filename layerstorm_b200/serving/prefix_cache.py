"""Prefix cache: a radix tree of frozen holder sequences.

A finished prompt leaves a *holder* (a forked, never-appending sequence) registered at
grid-aligned lengths; a new request whose prompt shares a prefix forks from the deepest holder
instead of prefilling those tokens again (copy-on-write pages).  Nodes exist only at multiples
of ``grid`` tokens (or the exact prompt body), so cache ON and OFF run the same chunk shapes and
give identical tokens.  Eviction is leaf-only, least-recently-used first, deepest first among
equals; the token budget counts unique (edge) tokens.  Models with recurrent state (KDA) can only
be forked at a holder's exact frontier.
Reference: PrefixCache in python/orchestrator/orchestrator.py:598-643,804-1272 (radix tree of frozen
holders, touch propagation, leaf-only LRU eviction, fork-with-evict-retry).
"""
from __future__ import annotations

import itertools
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple


@dataclass
class PrefixCacheConfig:
    enabled: bool = True
    grid: int = 64                    # node granularity in tokens
    max_tokens: int = 1 << 20         # budget over unique cached tokens
    max_holders: int = 64
    min_prefix: int = 64


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
        return holder

    def fork_from(self, tokens: List[int]) -> Tuple[Optional[int], int]:
        """New live sequence sharing the longest cached prefix: (seq id, prefix length)."""
        holder, n = self.lookup(tokens)
        if holder is None:
            return None, 0
        for attempt in range(2):
            try:
                return self.engine.fork_sequence(holder, n), n
            except Exception:  # noqa: BLE001
                if attempt or not self.evict_one(protect=holder):
                    break
        return None, 0

    def evict_one(self, protect: Optional[int] = None) -> bool:
        """Drop the least recently used leaf holder (deepest first among equals)."""
        if self.recurrent:
            cands = [(lu, -len(k), k) for k, (h, lu) in self.exact.items() if h != protect]
            if not cands:
                return False
            k = min(cands)[2]
            self.engine.free_sequence(self.exact.pop(k)[0])
            return True
        best = None
        for n in self._nodes():
            if n is self.root or n.children or n.holder is None or n.holder == protect:
                continue
            if best is None or (n.last_used, -n.depth) < (best.last_used, -best.depth):
                best = n
        if best is None:
            return False
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
