"""OpenAI-compatible HTTP API: /health, /v1/models, /v1/completions, /v1/chat/completions.

Streaming uses server-sent events with comment heartbeats while a long prefill produces no
data; admission is a bounded FIFO (beyond it: 503 + Retry-After); a client disconnect cancels
the request.  Chat requests go through the chat template, optional tool-call and reasoning
parsers and optional guided decoding (``response_format``).
Reference: python/server/http_server.py:574-589 (routes), :379-451 (disconnect cancel), :1196
(bounded admission), python/server/streaming.py (SSE + heartbeat).
"""
from __future__ import annotations

import asyncio
import json
import queue
import time
import uuid
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from fastapi import FastAPI, Request
from fastapi.responses import JSONResponse, StreamingResponse

from .guided import make_logit_mask
from .orchestrator import InferenceRequest, Orchestrator, SamplingParams
from .parsers import StreamingReasoningSplitter, get_reasoning_parser, get_tool_parser
from .tokenizer import ChatTemplateRenderer, IncrementalDetokenizer, TokenizerWrapper


@dataclass
class ServerConfig:
    model_name: str = "layerstorm-b200"
    max_concurrent: int = 1
    max_queued_requests: int = 16
    sse_heartbeat_seconds: float = 10.0
    max_sequence_length: int = 8192
    default_max_tokens: int = 256
    tool_call_parser: Optional[str] = None
    enable_auto_tool_choice: bool = False
    reasoning_parser: Optional[str] = None
    reasoning_config: Optional[dict] = None
    retry_after_seconds: int = 5


def _error(status: int, message: str, etype: str = "invalid_request_error", headers: Optional[dict] = None):
    return JSONResponse({"error": {"message": message, "type": etype, "code": status}}, status_code=status, headers=headers)


def sampling_from_body(body: dict, cfg: ServerConfig) -> SamplingParams:
    stop = body.get("stop") or []
    if isinstance(stop, str):
        stop = [stop]
    lp = body.get("logprobs")
    if isinstance(lp, bool):
        lp = int(body.get("top_logprobs") or 1) if lp else 0
    mt = body.get("max_completion_tokens") or body.get("max_tokens") or cfg.default_max_tokens
    return SamplingParams(max_tokens=int(mt), temperature=float(body.get("temperature", 0.0) or 0.0), top_k=int(body.get("top_k", 0) or 0),
                          top_p=float(body.get("top_p", 1.0) or 1.0), seed=body.get("seed"), stop=list(stop),
                          stop_token_ids=list(body.get("stop_token_ids") or []), logprobs=int(lp or 0),
                          ignore_eos=bool(body.get("ignore_eos", False)))


class LayerStormServer:
    def __init__(self, orch: Orchestrator, tokenizer: TokenizerWrapper, cfg: Optional[ServerConfig] = None,
                 template: Optional[ChatTemplateRenderer] = None):
        self.orch, self.tok, self.cfg = orch, tokenizer, cfg or ServerConfig()
        self.template = template or ChatTemplateRenderer(tokenizer.chat_template)
        self.tool_parser = get_tool_parser(self.cfg.tool_call_parser) if self.cfg.tool_call_parser else None
        self.reasoning = get_reasoning_parser(self.cfg.reasoning_parser, self.cfg.reasoning_config) if self.cfg.reasoning_parser else None
        self.inflight = 0
        self.started = time.time()
        self.app = FastAPI(title="layerstorm-b200")
        self.app.get("/health")(self.health)
        self.app.get("/v1/models")(self.models)
        self.app.post("/v1/completions")(self.completions)
        self.app.post("/v1/chat/completions")(self.chat_completions)

    # ---- simple routes ----
    async def health(self):
        # a multi-process server is healthy only while every rank is alive (set by the CLI: () -> {rank: reason} of failed ranks)
        failed = self.failed_ranks() if getattr(self, "failed_ranks", None) else None
        if failed:
            return _error(503, "rank(s) down: " + "; ".join(f"{r}: {why}" for r, why in sorted(failed.items())), "server_error")
        if getattr(self.orch, "gpu_fatal", None):
            return _error(503, "gpu_fatal: " + self.orch.gpu_fatal, "server_error")
        # engine-side numbers come from the orchestrator's published state block (seqlock snapshot written by the serving thread)
        state = self.orch.published_state() if hasattr(self.orch, "published_state") else {}
        return {"status": "ok", "uptime_s": round(time.time() - self.started, 1), "queued": self.orch.queued(), "served": self.orch.served,
                "speculation": self._speculation_state(),
                "engine": state, "admission_waits": getattr(self.orch, "admission_waits", 0), "preemptions": getattr(self.orch, "preemptions", 0)}

    def _speculation_state(self) -> dict:
        """What the draft side is doing (plain attribute reads of numbers the serving thread writes): per-source acceptance estimates and
        the source chosen last (draft combiner), the depth policy's acceptance and how many rounds it left to plain decoding, rounds
        drafted inside a think block; empty without a draft."""
        d = getattr(self.orch, "draft", None)
        if d is None:
            return {}
        out = {"depth": getattr(self.orch, "gamma", 0), "think_rounds": getattr(self.orch, "think_rounds", 0)}
        if hasattr(d, "sources"):
            out["sources"] = {s.name: round(float(s.acceptance), 3) for s in d.sources}
            out["last_source"] = d.last.name if getattr(d, "last", None) is not None else None
        pol = getattr(self.orch, "depth_policy", None)
        if pol is not None:
            out["acceptance"] = round(float(pol.acceptance), 3)
            out["plain_rounds"] = int(pol.plain_rounds)
        return out

    async def models(self):
        return {"object": "list", "data": [{"id": self.cfg.model_name, "object": "model", "created": int(self.started), "owned_by": "layerstorm-b200",
                                            "max_model_len": self.cfg.max_sequence_length}]}

    # ---- admission ----
    def _admit(self):
        if getattr(self.orch, "gpu_fatal", None):
            return _error(503, "gpu_fatal: " + self.orch.gpu_fatal, "server_error")
        if self.inflight >= self.cfg.max_concurrent + self.cfg.max_queued_requests:
            return _error(503, "server busy: generation queue is full", "server_overloaded", {"Retry-After": str(self.cfg.retry_after_seconds)})
        self.inflight += 1
        return None

    def _release(self, *_):
        self.inflight = max(0, self.inflight - 1)

    # ---- request plumbing ----
    def _submit(self, prompt_ids: List[int], params: SamplingParams, logit_mask=None):
        q: "queue.Queue" = queue.Queue()
        rid = "req-" + uuid.uuid4().hex[:16]
        req = InferenceRequest(rid, prompt_ids, params, on_token=lambda t, info: q.put(("tok", t, info)),
                               on_done=lambda r: q.put(("done", r, None)), logit_mask=logit_mask)
        self.orch.submit_request(req)
        return req, q

    async def _next_event(self, q: "queue.Queue", timeout: float):
        loop = asyncio.get_running_loop()
        try:
            return await loop.run_in_executor(None, lambda: q.get(timeout=timeout))
        except queue.Empty:
            return None

    async def _collect(self, request: Request, req: InferenceRequest, q):
        """Non-streaming: wait for completion, cancelling on client disconnect."""
        lps = []
        while True:
            ev = await self._next_event(q, 0.25)
            if ev is None:
                if await request.is_disconnected():
                    self.orch.cancel_request(req.request_id)
                continue
            if ev[0] == "tok":
                if ev[2] is not None:
                    lps.append((ev[1], ev[2]))
            else:
                return lps

    def _usage(self, req: InferenceRequest) -> dict:
        u = {"prompt_tokens": len(req.prompt_ids), "completion_tokens": len(req.output_ids),
             "total_tokens": len(req.prompt_ids) + len(req.output_ids)}
        if req.stats.cached_tokens:
            u["prompt_tokens_details"] = {"cached_tokens": req.stats.cached_tokens}
        return u

    def _logprobs_obj(self, lps) -> Optional[dict]:
        if not lps:
            return None
        return {"content": [{"token": self.tok.decode([t]), "logprob": info["logprob"],
                             "top_logprobs": [{"token": self.tok.decode([i]), "logprob": v} for i, v in info["top"]]} for t, info in lps]}

    def _strip_stop(self, text: str, stops: List[str]) -> str:
        for s in stops:
            if s and s in text:
                text = text.split(s, 1)[0]
        return text

    # ---- /v1/completions ----
    async def completions(self, request: Request):
        try:
            body = await request.json()
        except Exception:  # noqa: BLE001
            return _error(400, "request body is not valid JSON")
        prompt = body.get("prompt")
        if isinstance(prompt, list) and prompt and isinstance(prompt[0], int):
            ids = [int(t) for t in prompt]
        elif isinstance(prompt, str):
            ids = self.tok.encode(prompt)
        else:
            return _error(400, "`prompt` must be a string or a list of token ids")
        if not ids:
            return _error(400, "empty prompt")
        if len(ids) > self.cfg.max_sequence_length:
            return _error(400, f"prompt has {len(ids)} tokens; the limit is {self.cfg.max_sequence_length}")
        busy = self._admit()
        if busy is not None:
            return busy
        params = sampling_from_body(body, self.cfg)
        req, q = self._submit(ids, params)
        cid, created = "cmpl-" + uuid.uuid4().hex[:24], int(time.time())
        if body.get("stream"):
            return StreamingResponse(self._stream(request, req, q, cid, created, chat=False), media_type="text/event-stream",
                                     background=_Bg(self._release))
        try:
            lps = await self._collect(request, req, q)
        finally:
            self._release()
        if req.error:
            return _error(500, req.error, "engine_error")
        text = self._strip_stop(self.tok.decode(req.output_ids), params.stop)
        return {"id": cid, "object": "text_completion", "created": created, "model": self.cfg.model_name,
                "choices": [{"index": 0, "text": text, "finish_reason": req.finish_reason, "logprobs": self._logprobs_obj(lps)}],
                "usage": self._usage(req)}

    # ---- /v1/chat/completions ----
    async def chat_completions(self, request: Request):
        try:
            body = await request.json()
        except Exception:  # noqa: BLE001
            return _error(400, "request body is not valid JSON")
        messages = body.get("messages")
        if not isinstance(messages, list) or not messages:
            return _error(400, "`messages` must be a non-empty list")
        tools = body.get("tools")
        try:
            text = self.template.render(messages, tools=tools, add_generation_prompt=True, **(body.get("chat_template_kwargs") or {}))
        except Exception as exc:  # noqa: BLE001
            return _error(400, f"chat template error: {exc}")
        ids = self.tok.encode(text)
        if len(ids) > self.cfg.max_sequence_length:
            return _error(400, f"prompt has {len(ids)} tokens; the limit is {self.cfg.max_sequence_length}")
        mask = None
        rf = body.get("response_format")
        if rf and rf.get("type") in ("json_object", "json_schema"):
            try:
                mask = make_logit_mask(self.tok, rf)
            except Exception as exc:  # noqa: BLE001
                return _error(400, f"unsupported response_format: {exc}")
        busy = self._admit()
        if busy is not None:
            return busy
        params = sampling_from_body(body, self.cfg)
        req, q = self._submit(ids, params, mask)
        cid, created = "chatcmpl-" + uuid.uuid4().hex[:24], int(time.time())
        use_tools = bool(tools) and self.tool_parser is not None and (
            body.get("tool_choice") not in (None, "auto") or self.cfg.enable_auto_tool_choice) and body.get("tool_choice") != "none"
        if body.get("stream"):
            return StreamingResponse(self._stream(request, req, q, cid, created, chat=True, use_tools=use_tools),
                                     media_type="text/event-stream", background=_Bg(self._release))
        try:
            lps = await self._collect(request, req, q)
        finally:
            self._release()
        if req.error:
            return _error(500, req.error, "engine_error")
        out = self._strip_stop(self.tok.decode(req.output_ids), params.stop)
        msg: Dict[str, Any] = {"role": "assistant", "content": out}
        if self.reasoning is not None:
            r, c = self.reasoning.parse(out)
            msg["content"] = c
            if r is not None:
                msg["reasoning_content"] = r
        finish = req.finish_reason
        if use_tools:
            rest, calls = self.tool_parser.parse(msg["content"] or "")
            if calls:
                msg["content"] = rest or None
                msg["tool_calls"] = [c.to_openai() for c in calls]
                finish = "tool_calls"
        return {"id": cid, "object": "chat.completion", "created": created, "model": self.cfg.model_name,
                "choices": [{"index": 0, "message": msg, "finish_reason": finish, "logprobs": self._logprobs_obj(lps)}],
                "usage": self._usage(req)}

    # ---- SSE ----
    async def _stream(self, request: Request, req: InferenceRequest, q, cid: str, created: int, chat: bool, use_tools: bool = False):
        detok = IncrementalDetokenizer(self.tok)
        splitter = StreamingReasoningSplitter(self.reasoning) if (chat and self.reasoning is not None) else None
        obj = "chat.completion.chunk" if chat else "text_completion"
        last = time.time()
        held = ""          # with tool parsing the content is held back and emitted at the end

        def chunk(delta: Optional[dict] = None, text: Optional[str] = None, finish: Optional[str] = None, usage: Optional[dict] = None):
            ch: Dict[str, Any] = {"index": 0, "finish_reason": finish}
            if chat:
                ch["delta"] = delta or {}
            else:
                ch["text"] = text or ""
            d = {"id": cid, "object": obj, "created": created, "model": self.cfg.model_name, "choices": [ch]}
            if usage:
                d["usage"] = usage
            return "data: " + json.dumps(d, ensure_ascii=False) + "\n\n"

        if chat:
            yield chunk({"role": "assistant", "content": ""})
        while True:
            ev = await self._next_event(q, 0.25)
            if ev is None:
                if await request.is_disconnected():
                    self.orch.cancel_request(req.request_id)
                    return
                hb = self.cfg.sse_heartbeat_seconds
                if hb > 0 and time.time() - last >= hb:
                    last = time.time()
                    yield ": keep-alive\n\n"
                continue
            last = time.time()
            if ev[0] == "tok":
                piece = detok.push(ev[1])
                if not piece:
                    continue
                if not chat:
                    yield chunk(text=piece)
                    continue
                r_d, c_d = splitter.push(piece) if splitter else ("", piece)
                if r_d:
                    yield chunk({"reasoning_content": r_d})
                if c_d:
                    if use_tools:
                        held += c_d
                    else:
                        yield chunk({"content": c_d})
                continue
            finish = req.finish_reason
            if req.error:
                yield "data: " + json.dumps({"error": {"message": req.error, "type": "engine_error"}}) + "\n\n"
            elif chat and use_tools:
                rest, calls = self.tool_parser.parse(held)
                if rest:
                    yield chunk({"content": rest})
                if calls:
                    yield chunk({"tool_calls": [dict(c.to_openai(), index=i) for i, c in enumerate(calls)]})
                    finish = "tool_calls"
            yield chunk(finish=finish, usage=self._usage(req)) if chat else chunk(text="", finish=finish, usage=self._usage(req))
            yield "data: [DONE]\n\n"
            return

    def run(self, host: str = "127.0.0.1", port: int = 8000, log_level: str = "info"):
        import uvicorn
        uvicorn.run(self.app, host=host, port=port, log_level=log_level)


class _Bg:
    """Starlette background task shim: runs after the streaming response finishes."""

    def __init__(self, fn):
        self.fn = fn

    async def __call__(self):
        self.fn()
