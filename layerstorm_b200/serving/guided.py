"""Guided decoding for ``response_format`` (json_object / json_schema): a per-step mask of the
token ids that keep the output a valid prefix.

With a HuggingFace tokenizer the mask comes from xgrammar (compiled grammar + token bitmask), as
in the reference's structural-tag guided decoding.  With the built-in byte tokenizer a small JSON
pushdown automaton checks every byte token directly.  The mask composes with sampling and with
speculation because it is applied to the logits before the sampling transform.
Reference: python/server guided decoding (xgrammar), python/orchestrator/orchestrator.py:3736-3740.
"""
from __future__ import annotations

import json
from typing import Callable, List, Optional

import torch


class JsonPrefixValidator:
    """Incremental validator: feed characters; ``ok`` stays True while the text is a prefix of some
    JSON value; ``complete`` is True when a full top-level value has been read."""

    WS = " \t\n\r"

    def __init__(self, require_object: bool = True):
        self.stack: List[str] = []          # 'obj_key', 'obj_colon', 'obj_val', 'obj_next', 'arr_val', 'arr_next'
        self.mode = "value"                 # value | string | escape | unicode | number | literal | done
        self.lit_rest = ""
        self.uni_left = 0
        self.str_is_key = False
        self.num = ""
        self.ok = True
        self.complete = False
        self.require_object = require_object
        self.started = False

    def copy(self) -> "JsonPrefixValidator":
        c = JsonPrefixValidator(self.require_object)
        c.__dict__.update({k: (list(v) if isinstance(v, list) else v) for k, v in self.__dict__.items()})
        return c

    def _value_done(self):
        if not self.stack:
            self.mode, self.complete = "done", True
            return
        top = self.stack[-1]
        if top == "obj_val":
            self.stack[-1] = "obj_next"
        elif top == "arr_val":
            self.stack[-1] = "arr_next"
        self.mode = "between"

    @staticmethod
    def _num_prefix_ok(s: str) -> bool:
        import re
        return re.fullmatch(r"-?(0|[1-9]\d*)?(\.\d*)?([eE][+-]?\d*)?", s) is not None and s not in ("", )

    @staticmethod
    def _num_complete(s: str) -> bool:
        import re
        return re.fullmatch(r"-?(0|[1-9]\d*)(\.\d+)?([eE][+-]?\d+)?", s) is not None

    def feed(self, ch: str) -> bool:
        if not self.ok:
            return False
        m = self.mode
        if m == "number":
            if ch in "0123456789+-.eE" and self._num_prefix_ok(self.num + ch):
                self.num += ch
                return True
            if not self._num_complete(self.num):
                self.ok = False
                return False
            self._value_done()
            m = self.mode           # fall through with the same character
        if m == "string":
            if ch == "\\":
                self.mode = "escape"
            elif ch == '"':
                if self.str_is_key:
                    self.stack[-1] = "obj_colon"
                    self.mode = "between"
                else:
                    self._value_done()
            elif ord(ch) < 0x20:
                self.ok = False
            return self.ok
        if m == "escape":
            if ch == "u":
                self.mode, self.uni_left = "unicode", 4
            elif ch in '"\\/bfnrt':
                self.mode = "string"
            else:
                self.ok = False
            return self.ok
        if m == "unicode":
            if ch in "0123456789abcdefABCDEF":
                self.uni_left -= 1
                if self.uni_left == 0:
                    self.mode = "string"
            else:
                self.ok = False
            return self.ok
        if m == "literal":
            if self.lit_rest and ch == self.lit_rest[0]:
                self.lit_rest = self.lit_rest[1:]
                if not self.lit_rest:
                    self._value_done()
            else:
                self.ok = False
            return self.ok
        if ch in self.WS:
            return True
        if m == "done":
            self.ok = False
            return False
        if m == "between":
            top = self.stack[-1]
            if top == "obj_key":
                if ch == '"':
                    self.mode, self.str_is_key = "string", True
                elif ch == "}" and self.stack[-1] == "obj_key" and getattr(self, "_empty_ok", False):
                    self.stack.pop(); self._empty_ok = False; self._value_done()
                else:
                    self.ok = False
            elif top == "obj_colon":
                if ch == ":":
                    self.stack[-1] = "obj_val"; self.mode = "value"
                else:
                    self.ok = False
            elif top == "obj_next":
                if ch == ",":
                    self.stack[-1] = "obj_key"; self._empty_ok = False
                elif ch == "}":
                    self.stack.pop(); self._value_done()
                else:
                    self.ok = False
            elif top == "arr_next":
                if ch == ",":
                    self.stack[-1] = "arr_val"; self.mode = "value"; self._arr_empty_ok = False
                elif ch == "]":
                    self.stack.pop(); self._value_done()
                else:
                    self.ok = False
            return self.ok
        # mode == "value"
        if not self.started:
            self.started = True
            if self.require_object and ch != "{":
                self.ok = False
                return False
        if ch == "{":
            self.stack.append("obj_key"); self.mode = "between"; self._empty_ok = True
        elif ch == "[":
            self.stack.append("arr_val"); self.mode = "value"; self._arr_empty_ok = True
        elif ch == "]" and self.stack and self.stack[-1] == "arr_val" and getattr(self, "_arr_empty_ok", False):
            self.stack.pop(); self._arr_empty_ok = False; self._value_done()
        elif ch == '"':
            self.mode, self.str_is_key = "string", False
        elif ch in "-0123456789":
            self.mode, self.num = "number", ch
        elif ch in "tfn":
            self.mode, self.lit_rest = "literal", {"t": "rue", "f": "alse", "n": "ull"}[ch]
        else:
            self.ok = False
        if ch != "[":
            self._arr_empty_ok = False
        return self.ok

    def feed_text(self, s: str) -> bool:
        for ch in s:
            if not self.feed(ch):
                return False
        return True


def make_logit_mask(tokenizer, response_format: dict) -> Callable[[List[int]], Optional[torch.Tensor]]:
    """Returns mask_fn(output_ids) -> bool tensor [vocab] of allowed next tokens (None = no limit)."""
    if getattr(tokenizer, "tok", None) is not None:
        return _xgrammar_mask(tokenizer, response_format)
    vocab = tokenizer.vocab_size
    pieces = [tokenizer.decode([i]) if i < 256 else "" for i in range(vocab)]
    eos = set(tokenizer.eos_token_ids)

    def mask_fn(output_ids: List[int]) -> Optional[torch.Tensor]:
        v = JsonPrefixValidator(require_object=True)
        v.feed_text(tokenizer.decode(output_ids))
        m = torch.zeros(vocab, dtype=torch.bool)
        if v.complete:
            for e in eos:
                m[e] = True
            return m
        for i, p in enumerate(pieces):
            if p and p != "�" and v.copy().feed_text(p):
                m[i] = True
        if not m.any():
            return None
        return m
    return mask_fn


def _xgrammar_mask(tokenizer, response_format: dict):
    import xgrammar as xgr
    vocab = tokenizer.vocab_size
    enc = [tokenizer.tok.id_to_token(i) or "" for i in range(vocab)]
    info = xgr.TokenizerInfo(enc, stop_token_ids=list(tokenizer.eos_token_ids) or None)
    comp = xgr.GrammarCompiler(info)
    if response_format.get("type") == "json_schema":
        schema = response_format.get("json_schema", {}).get("schema") or response_format.get("schema") or {}
        grammar = comp.compile_json_schema(json.dumps(schema))
    else:
        grammar = comp.compile_builtin_json_grammar()
    matcher = xgr.GrammarMatcher(grammar)
    state = {"n": 0}
    bitmask = xgr.allocate_token_bitmask(1, vocab)

    def mask_fn(output_ids: List[int]) -> Optional[torch.Tensor]:
        for t in output_ids[state["n"]:]:
            matcher.accept_token(int(t))
        state["n"] = len(output_ids)
        if matcher.is_terminated():
            return None
        matcher.fill_next_token_bitmask(bitmask)
        bits = bitmask[0].to(torch.int64)
        idx = torch.arange(vocab)
        return ((bits[idx // 32] >> (idx % 32)) & 1).bool()
    return mask_fn
