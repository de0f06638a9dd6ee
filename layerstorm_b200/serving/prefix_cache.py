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
    tokens: Tuple[int, ...]           # edge label (tokens since the parent)
    depth: int                        # total tokens from the root
    holder: Optional[int] = None      # engine sequence id holding KV for [0, depth)
    children: Dict[int, "_Node"] = field(default_factory=dict)
    parent: Optional["_Node"] = None
    last_used: int = 0


class PrefixCache:
    def __init__(self, engine, cfg: Optional[PrefixCacheConfig] = None):
        self.engine, self.cfg = engine, cfg or PrefixCacheConfig()
        self.root = _Node((), 0)
        self._clock = itertools.count(1)
        self.hits = self.misses = self.hit_tokens = 0

    # ---- queries ----
    def _walk(self, tokens: List[int]) -> Tuple[_Node, int]:
        """Deepest node whose path is a prefix of ``tokens``; returns (node, matched_len)."""
        node, pos = self.root, 0
        while pos < len(tokens):
            ch = node.children.get(tokens[pos])
            if ch is None:
                break
            n = len(ch.tokens)
            if tuple(tokens[pos: pos + n]) != ch.tokens:
                break
            node, pos = ch, pos + n
        return node, pos

    def lookup(self, tokens: List[int]) -> Tuple[Optional[int], int]:
        """(holder sequence id, prefix length) of the longest usable cached prefix, or (None, 0).
        At least one prompt token is always left to prefill so the request gets fresh logits."""
        if not self.cfg.enabled:
            return None, 0
        node, pos = self._walk(tokens)
        while node is not self.root and (node.holder is None or node.depth >= len(tokens)):
            node = node.parent
        if node is self.root or node.depth < self.cfg.min_prefix:
            self.misses += 1
            return None, 0
        t = next(self._clock)
        n = node
        while n is not None:            # touch propagates to ancestors
            n.last_used = t
            n = n.parent
        self.hits += 1
        self.hit_tokens += node.depth
        return node.holder, node.depth

    def total_tokens(self) -> int:
        tot, stack = 0, [self.root]
        while stack:
            n = stack.pop()
            tot += len(n.tokens)
            stack.extend(n.children.values())
        return tot

    def holders(self) -> int:
        cnt, stack = 0, [self.root]
        while stack:
            n = stack.pop()
            cnt += n.holder is not None
            stack.extend(n.children.values())
        return cnt

    # ---- updates ----
    def register(self, seq_id: int, tokens: List[int]) -> Optional[int]:
        """Freeze a copy of ``seq_id`` (whose KV covers ``tokens``) at the largest grid-aligned
        length; returns the holder id or None (too short / already cached / no room)."""
        if not self.cfg.enabled:
            return None
        depth = (len(tokens) // self.cfg.grid) * self.cfg.grid
        recurrent = getattr(self.engine, "has_recurrent_state", False)
        if recurrent:
            depth = len(tokens)          # recurrent state exists only at the frontier
        if depth < self.cfg.min_prefix:
            return None
        node, pos = self._walk(tokens[:depth])
        if pos == depth and node.holder is not None:
            node.last_used = next(self._clock)
            return node.holder
        while (self.total_tokens() + (depth - pos) > self.cfg.max_tokens or self.holders() >= self.cfg.max_holders):
            if not self.evict_one():
                return None
            node, pos = self._walk(tokens[:depth])
        try:
            holder = self.engine.fork_sequence(seq_id, depth)
        except Exception:  # noqa: BLE001 - no slot / pool: caching is best effort
            return None
        if pos < depth:
            child = _Node(tuple(tokens[pos:depth]), depth, parent=node)
            node.children[tokens[pos]] = child
            node = child
        node.holder = holder
        node.last_used = next(self._clock)
        return holder

    def fork_from(self, tokens: List[int]) -> Tuple[Optional[int], int]:
        """New live sequence sharing the longest cached prefix: (seq id, prefix length)."""
        holder, n = self.lookup(tokens)
        if holder is None:
            return None, 0
        try:
            return self.engine.fork_sequence(holder, n), n
        except Exception:  # noqa: BLE001
            if self.evict_one(protect=holder):
                try:
                    return self.engine.fork_sequence(holder, n), n
                except Exception:  # noqa: BLE001
                    pass
            return None, 0

    def evict_one(self, protect: Optional[int] = None) -> bool:
        """Drop the least recently used leaf holder (deepest first among equals)."""
        best, stack = None, [self.root]
        while stack:
            n = stack.pop()
            stack.extend(n.children.values())
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
            del n.parent.children[n.tokens[0]]
            n = n.parent
        return True

    def clear(self):
        while self.evict_one():
            pass
