"""Prompt-lookup drafting: propose the continuation that followed the most recent earlier occurrence
of the current n-gram suffix.  Costs no model forward, so it is always worth trying first on
copy-heavy workloads (code edits, RAG answers, summaries).
Reference: the ``speculation.prompt_lookup`` method (config/schema.json: min/max n-gram size, max
continuation length; python/orchestrator/prompt_lookup.py).
"""
from __future__ import annotations

from typing import Dict, List, Sequence, Tuple


class PromptLookupDraft:
    def __init__(self, min_ngram: int = 2, max_ngram: int = 4, max_continuation: int = 5):
        assert 1 <= min_ngram <= max_ngram
        self.min_n, self.max_n, self.max_cont = min_ngram, max_ngram, max_continuation
        self.hits = 0
        self.calls = 0

    def propose(self, context: Sequence[int], gamma: int) -> List[int]:
        """Longest n-gram first; among matches of equal length the most recent one wins."""
        self.calls += 1
        g = min(gamma, self.max_cont)
        n_ctx = len(context)
        if g <= 0 or n_ctx < self.min_n + 1:
            return []
        for n in range(min(self.max_n, n_ctx - 1), self.min_n - 1, -1):
            suffix = tuple(context[n_ctx - n:])
            for start in range(n_ctx - n - 1, -1, -1):
                if tuple(context[start:start + n]) == suffix:
                    cont = list(context[start + n:start + n + g])
                    if cont:
                        self.hits += 1
                        return cont
        return []


class IncrementalPromptLookup(PromptLookupDraft):
    """Same proposals with an n-gram -> last-position index kept across calls for one sequence, so a
    long context costs O(new tokens) per call instead of a rescan."""

    def __init__(self, min_ngram: int = 2, max_ngram: int = 4, max_continuation: int = 5):
        super().__init__(min_ngram, max_ngram, max_continuation)
        self.index: Dict[Tuple[int, ...], int] = {}
        self.indexed = 0
        self.tokens: List[int] = []

    def reset(self):
        self.index.clear()
        self.indexed = 0
        self.tokens = []

    def _extend(self, context: Sequence[int]):
        if len(context) < len(self.tokens) or list(context[:len(self.tokens)]) != self.tokens:
            self.reset()
        self.tokens = list(context)
        # index every n-gram that is followed by at least one token, i.e. ends before the last position
        end = len(self.tokens) - 1
        for pos in range(self.indexed, end):
            for n in range(self.min_n, self.max_n + 1):
                if pos + 1 - n >= 0:
                    self.index[tuple(self.tokens[pos + 1 - n:pos + 1])] = pos + 1     # position of the continuation
        self.indexed = max(self.indexed, end)

    def propose(self, context: Sequence[int], gamma: int) -> List[int]:
        self.calls += 1
        g = min(gamma, self.max_cont)
        if g <= 0 or len(context) < self.min_n + 1:
            return []
        self._extend(context)
        for n in range(min(self.max_n, len(context) - 1), self.min_n - 1, -1):
            at = self.index.get(tuple(context[len(context) - n:]))
            if at is not None:
                cont = self.tokens[at:at + g]
                if cont:
                    self.hits += 1
                    return list(cont)
        return []
