"""Tokenizer wrapper, special-token detection and chat-template rendering.

``TokenizerWrapper`` loads a HuggingFace ``tokenizer.json`` directory through the ``tokenizers``
library when one is given and otherwise falls back to a byte-level tokenizer (ids 0..255 + a few
specials), which keeps the serving stack usable with random-init models and in CPU tests.
Locator precedence: explicit path > ``<weights>/tokenizer.json`` > parent directory.
Reference: python/tokenizer/* (HF wrapper, special-token detection, jinja chat template, locator).
"""
from __future__ import annotations

import json
import os
from typing import Dict, List, Optional, Sequence


class ByteTokenizer:
    """256 byte tokens + <bos>=256, <eos>=257, <pad>=258."""
    vocab_size = 259
    bos_id, eos_id, pad_id = 256, 257, 258

    def encode(self, text: str) -> List[int]:
        return list(text.encode("utf-8"))

    def decode(self, ids: Sequence[int]) -> str:
        return bytes(i for i in ids if 0 <= i < 256).decode("utf-8", errors="replace")


def resolve_tokenizer_dir(explicit: Optional[str], weights_path: Optional[str]) -> Optional[str]:
    """explicit path ('auto' = detect) > next to the weights > the weights' parent directory."""
    cands = []
    if explicit and explicit != "auto":
        cands.append(explicit)
    if weights_path:
        base = weights_path if os.path.isdir(weights_path) else os.path.dirname(weights_path)
        cands += [base, os.path.dirname(base)]
    for c in cands:
        if c and os.path.exists(os.path.join(c, "tokenizer.json")):
            return c
    return None


class TokenizerWrapper:
    def __init__(self, path: Optional[str] = None, vocab_limit: Optional[int] = None):
        self.path = path
        self.tok = None
        self.byte = None
        self.special: Dict[str, int] = {}
        self.eos_token_ids: List[int] = []
        self.chat_template: Optional[str] = None
        self.vocab_limit = vocab_limit
        if path and os.path.exists(os.path.join(path, "tokenizer.json")):
            from tokenizers import Tokenizer
            self.tok = Tokenizer.from_file(os.path.join(path, "tokenizer.json"))
            self._detect_specials(path)
        else:
            self.byte = ByteTokenizer()
            self.eos_token_ids = [self.byte.eos_id]
            self.special = {"<bos>": 256, "<eos>": 257, "<pad>": 258}

    def _detect_specials(self, path: str):
        cfgp = os.path.join(path, "tokenizer_config.json")
        cfg = json.load(open(cfgp)) if os.path.exists(cfgp) else {}
        for tid, ent in (cfg.get("added_tokens_decoder") or {}).items():
            if ent.get("special"):
                self.special[ent["content"]] = int(tid)
        eos = cfg.get("eos_token")
        eos = eos.get("content") if isinstance(eos, dict) else eos
        if eos and self.tok.token_to_id(eos) is not None:
            self.eos_token_ids = [self.tok.token_to_id(eos)]
        gen = os.path.join(path, "generation_config.json")
        if os.path.exists(gen):
            e = json.load(open(gen)).get("eos_token_id")
            if e is not None:
                self.eos_token_ids = sorted(set(self.eos_token_ids + (e if isinstance(e, list) else [e])))
        self.chat_template = cfg.get("chat_template")
        tp = os.path.join(path, "chat_template.jinja")
        if os.path.exists(tp):
            self.chat_template = open(tp).read()

    @property
    def vocab_size(self) -> int:
        return self.tok.get_vocab_size() if self.tok else self.byte.vocab_size

    def encode(self, text: str, add_special_tokens: bool = False) -> List[int]:
        ids = self.tok.encode(text, add_special_tokens=add_special_tokens).ids if self.tok else self.byte.encode(text)
        if self.vocab_limit:
            ids = [i % self.vocab_limit for i in ids]
        return ids

    def decode(self, ids: Sequence[int], skip_special_tokens: bool = True) -> str:
        if self.tok:
            return self.tok.decode(list(ids), skip_special_tokens=skip_special_tokens)
        return self.byte.decode(ids)


class IncrementalDetokenizer:
    """Streams text for a growing id list without splitting multi-byte characters: re-decodes a short
    tail window and emits only the stable new suffix."""

    def __init__(self, tok: TokenizerWrapper, window: int = 8):
        self.tok, self.window = tok, window
        self.ids: List[int] = []
        self.emitted = 0      # ids already fully emitted
        self.prefix_text = ""

    def push(self, tid: int) -> str:
        self.ids.append(tid)
        start = max(0, self.emitted - self.window)
        prev = self.tok.decode(self.ids[start:self.emitted])
        cur = self.tok.decode(self.ids[start:])
        if cur.endswith("�"):
            return ""          # incomplete UTF-8 sequence: wait for more ids
        self.emitted = len(self.ids)
        return cur[len(prev):]


DEFAULT_TEMPLATE = (
    "{% for m in messages %}<|{{ m['role'] }}|>\n{{ m['content'] if m['content'] is string else '' }}\n{% endfor %}"
    "{% if add_generation_prompt %}<|assistant|>\n{% endif %}")


class ChatTemplateRenderer:
    """Jinja chat template (from the tokenizer directory, or a minimal built-in)."""

    def __init__(self, template: Optional[str] = None):
        import jinja2
        from jinja2.sandbox import ImmutableSandboxedEnvironment
        env = ImmutableSandboxedEnvironment(trim_blocks=True, lstrip_blocks=True)
        env.globals["raise_exception"] = self._raise
        env.filters["tojson"] = lambda v, **kw: json.dumps(v, ensure_ascii=False, **{k: v2 for k, v2 in kw.items() if k == "indent"})
        self.template = env.from_string(template or DEFAULT_TEMPLATE)
        self._jinja2 = jinja2

    @staticmethod
    def _raise(msg):
        raise ValueError(msg)

    def render(self, messages: List[dict], tools: Optional[List[dict]] = None, add_generation_prompt: bool = True, **kwargs) -> str:
        return self.template.render(messages=messages, tools=tools, add_generation_prompt=add_generation_prompt, **kwargs)
