"""Output parsers: tool calls (-> OpenAI ``tool_calls``) and reasoning (-> ``reasoning_content``).

Tool-call formats:
  glm47        <tool_call>name\n<arg_key>k</arg_key>\n<arg_value>v</arg_value>...</tool_call>
  deepseek_v4  <｜tool▁call▁begin｜>name<｜tool▁sep｜>{json}<｜tool▁call▁end｜>   (also accepts the json-fenced form)
  hermes       <tool_call>{"name": ..., "arguments": {...}}</tool_call>
Reasoning formats:
  glm45 / deepseek_v4   <think> ... </think> answer   (markers overridable through a config)
Reference: python/server tool parsers (glm47, deepseek_v4, ...) and reasoning parsers (glm45, deepseek_v4).
"""
from __future__ import annotations

import json
import re
import uuid
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple


@dataclass
class ToolCall:
    name: str
    arguments: str                      # JSON text
    id: str = field(default_factory=lambda: "call_" + uuid.uuid4().hex[:24])

    def to_openai(self) -> dict:
        return {"id": self.id, "type": "function", "function": {"name": self.name, "arguments": self.arguments}}


def _coerce(v: str):
    s = v.strip()
    try:
        return json.loads(s)
    except Exception:  # noqa: BLE001 - plain string argument
        return v


class Glm47ToolParser:
    _CALL = re.compile(r"<tool_call>(.*?)</tool_call>", re.S)
    _KV = re.compile(r"<arg_key>(.*?)</arg_key>\s*<arg_value>(.*?)</arg_value>", re.S)

    def parse(self, text: str) -> Tuple[str, List[ToolCall]]:
        calls = []
        for body in self._CALL.findall(text):
            name = body.split("<arg_key>", 1)[0].strip().split("\n", 1)[0].strip()
            args = {k.strip(): _coerce(v) for k, v in self._KV.findall(body)}
            if name:
                calls.append(ToolCall(name, json.dumps(args, ensure_ascii=False)))
        return self._CALL.sub("", text).strip(), calls


class DeepseekV4ToolParser:
    _CALL = re.compile(r"<｜tool▁call▁begin｜>(.*?)<｜tool▁sep｜>(.*?)<｜tool▁call▁end｜>", re.S)
    _WRAP = re.compile(r"<｜tool▁calls▁begin｜>|<｜tool▁calls▁end｜>")

    def parse(self, text: str) -> Tuple[str, List[ToolCall]]:
        calls = []
        for name, body in self._CALL.findall(text):
            body = body.strip()
            m = re.search(r"```(?:json)?\s*(.*?)```", body, re.S)
            if m:
                body = m.group(1).strip()
            name = name.replace("function", "").strip() or name.strip()
            try:
                args = json.dumps(json.loads(body), ensure_ascii=False)
            except Exception:  # noqa: BLE001 - keep raw text when the model emitted invalid JSON
                args = body
            calls.append(ToolCall(name, args))
        rest = self._WRAP.sub("", self._CALL.sub("", text)).strip()
        return rest, calls


class HermesToolParser:
    _CALL = re.compile(r"<tool_call>\s*(\{.*?\})\s*</tool_call>", re.S)

    def parse(self, text: str) -> Tuple[str, List[ToolCall]]:
        calls = []
        for body in self._CALL.findall(text):
            try:
                o = json.loads(body)
                calls.append(ToolCall(o["name"], json.dumps(o.get("arguments", {}), ensure_ascii=False)))
            except Exception:  # noqa: BLE001
                continue
        return self._CALL.sub("", text).strip(), calls


TOOL_PARSERS = {"glm47": Glm47ToolParser, "glm45": Glm47ToolParser, "deepseek_v4": DeepseekV4ToolParser,
                "deepseek_v3": DeepseekV4ToolParser, "hermes": HermesToolParser}


def get_tool_parser(name: str):
    if name not in TOOL_PARSERS:
        raise ValueError(f"unknown tool-call parser {name!r} (known: {sorted(TOOL_PARSERS)})")
    return TOOL_PARSERS[name]()


class ReasoningParser:
    """Splits ``<think>reasoning</think>answer``.  With ``starts_in_reasoning`` the template already
    opened the block, so text before the end marker is reasoning even without a start marker."""

    def __init__(self, start: str = "<think>", end: str = "</think>", starts_in_reasoning: bool = False):
        self.start, self.end, self.starts_in_reasoning = start, end, starts_in_reasoning

    def parse(self, text: str) -> Tuple[Optional[str], str]:
        t = text
        if self.start and self.start in t:
            t = t.split(self.start, 1)[1]
            in_r = True
        else:
            in_r = self.starts_in_reasoning
        if not in_r:
            return None, text
        if self.end and self.end in t:
            r, c = t.split(self.end, 1)
            return r.strip(), c.lstrip("\n")
        return t.strip(), ""


class StreamingReasoningSplitter:
    """Incremental version for SSE: feed text deltas, get (reasoning_delta, content_delta)."""

    def __init__(self, parser: ReasoningParser):
        self.p = parser
        self.buf = ""
        self.state = "reasoning" if parser.starts_in_reasoning else "unknown"

    def push(self, delta: str) -> Tuple[str, str]:
        self.buf += delta
        r_out, c_out = "", ""
        while True:
            if self.state == "unknown":
                s = self.p.start
                if s and s in self.buf:
                    c_out += self.buf.split(s, 1)[0]
                    self.buf = self.buf.split(s, 1)[1]
                    self.state = "reasoning"
                    continue
                keep = self._partial_suffix(self.buf, s)
                c_out += self.buf[: len(self.buf) - keep]
                self.buf = self.buf[len(self.buf) - keep:]
                break
            if self.state == "reasoning":
                e = self.p.end
                if e and e in self.buf:
                    r_out += self.buf.split(e, 1)[0]
                    self.buf = self.buf.split(e, 1)[1].lstrip("\n")
                    self.state = "content"
                    continue
                keep = self._partial_suffix(self.buf, e)
                r_out += self.buf[: len(self.buf) - keep]
                self.buf = self.buf[len(self.buf) - keep:]
                break
            c_out += self.buf
            self.buf = ""
            break
        return r_out, c_out

    @staticmethod
    def _partial_suffix(buf: str, marker: str) -> int:
        if not marker:
            return 0
        for k in range(min(len(marker) - 1, len(buf)), 0, -1):
            if buf.endswith(marker[:k]):
                return k
        return 0


REASONING_PARSERS = {"glm45": dict(start="<think>", end="</think>"), "deepseek_v4": dict(start="<think>", end="</think>"),
                     "deepseek_r1": dict(start="<think>", end="</think>", starts_in_reasoning=True)}


def get_reasoning_parser(name: str, config: Optional[dict] = None) -> ReasoningParser:
    if name not in REASONING_PARSERS:
        raise ValueError(f"unknown reasoning parser {name!r} (known: {sorted(REASONING_PARSERS)})")
    kw = dict(REASONING_PARSERS[name])
    if config:
        if "reasoning_start_str" in config:
            kw["start"] = config["reasoning_start_str"]
        if "reasoning_end_str" in config:
            kw["end"] = config["reasoning_end_str"]
    return ReasoningParser(**kw)
