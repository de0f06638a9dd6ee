"""Request orchestrator: one generation loop on the main thread, fed by a thread-safe deque.

``submit_request`` is called from the HTTP thread; ``run`` / ``step`` serve requests in FIFO
order: prefix-cache lookup + fork, chunked prefill, then one of the decode arms (greedy,
sampled, speculative with a draft proposer, guided).  Tokens stream to the caller through the
request's ``on_token`` callback.  Pool exhaustion evicts a prefix holder and retries the same
chunk; cancellation is checked between steps.
Reference: Orchestrator in python/orchestrator/orchestrator.py:172-4257 (request deque,
_serve_next, _generate, decode arms, SpecRoundGovernor, RequestStats, _with_pool_evict_retry).
"""
from __future__ import annotations

import collections
import threading
import time
from dataclasses import dataclass, field
from typing import Callable, Deque, Dict, List, Optional, Sequence

import torch

from ..runtime.native import KvPoolExhausted
from .prefix_cache import PrefixCache, PrefixCacheConfig

import logging

log = logging.getLogger("layerstorm_b200.orchestrator")

_FATAL_MARKS = ("cuda error", "device-side assert", "illegal memory access", "illegal instruction", "unspecified launch failure",
                "misaligned address", "an uncorrectable ecc", "device has fallen off", "gpu is lost", "cudaerrorlaunch", "xid ")


def is_gpu_fatal(exc: BaseException) -> bool:
    """Whether an exception of a step means the device context is gone (a sticky CUDA error), as opposed to an error of the request
    (bad arguments, pool exhaustion, a bounded kernel wait that ran out - ``DeviceWaitError`` leaves the context usable).
    Reference: CMP_GPU_FATAL, emitted once per GPU when an event query returns an error (src/daemon/dispatch_completion.cpp:60-85)."""
    if type(exc).__name__ in ("AcceleratorError", "OutOfMemoryError") and "out of memory" in str(exc).lower():
        return False                             # an allocation failure is reported to the request, the context lives on
    if type(exc).__name__ == "DeviceWaitError":
        return False
    text = f"{type(exc).__name__}: {exc}".lower()
    return type(exc).__name__ == "AcceleratorError" or any(m in text for m in _FATAL_MARKS)


@dataclass
class SamplingParams:
    max_tokens: int = 128
    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 1.0
    seed: Optional[int] = None
    stop_token_ids: List[int] = field(default_factory=list)
    stop: List[str] = field(default_factory=list)
    logprobs: int = 0
    ignore_eos: bool = False

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0 or self.top_k == 1


@dataclass
class RequestStats:
    prompt_tokens: int = 0
    cached_tokens: int = 0
    completion_tokens: int = 0
    t_submit: float = 0.0
    t_start: float = 0.0
    t_first_token: float = 0.0
    t_done: float = 0.0
    spec_rounds: int = 0
    spec_accepted: int = 0
    pool_evict_retries: int = 0
    preemptions: int = 0                 # times the request gave its KV pages back in mid-decode and joined again
    moe_degraded_steps: int = 0        # engine steps of the DELIVERED attempt that ran without an expert the router selected (fetch deadline)
    degraded_retries: int = 0          # times the request was run again because its prefill was degraded (0 = served first try)

    @property
    def ttft_s(self) -> float:
        return self.t_first_token - self.t_start if self.t_first_token else 0.0

    @property
    def decode_tok_s(self) -> float:
        dt = self.t_done - self.t_first_token
        return (self.completion_tokens - 1) / dt if dt > 0 and self.completion_tokens > 1 else 0.0


@dataclass
class InferenceRequest:
    request_id: str
    prompt_ids: List[int]
    params: SamplingParams = field(default_factory=SamplingParams)
    on_token: Optional[Callable[[int, Optional[dict]], None]] = None      # (token id, logprob info)
    on_done: Optional[Callable[["InferenceRequest"], None]] = None
    logit_mask: Optional[Callable[[List[int]], Optional[torch.Tensor]]] = None   # guided decoding: allowed-token mask
    output_ids: List[int] = field(default_factory=list)
    finish_reason: Optional[str] = None
    error: Optional[str] = None
    cancelled: threading.Event = field(default_factory=threading.Event)
    done: threading.Event = field(default_factory=threading.Event)
    stats: RequestStats = field(default_factory=RequestStats)


def splitmix64(seed: int, pos: int) -> int:
    """Per-position sampling seed: the same request seed gives the same trajectory whether tokens
    are produced one at a time or accepted in speculative batches."""
    z = (seed + 0x9E3779B97F4A7C15 * (pos + 1)) & 0xFFFFFFFFFFFFFFFF
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & 0xFFFFFFFFFFFFFFFF
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & 0xFFFFFFFFFFFFFFFF
    return z ^ (z >> 31)


def target_probs(logits: torch.Tensor, p: SamplingParams) -> torch.Tensor:
    """Target distribution after temperature / top-k / top-p."""
    lg = logits.float() / max(p.temperature, 1e-6)
    if p.top_k and p.top_k < lg.numel():
        kth = torch.topk(lg, p.top_k).values[-1]
        lg = torch.where(lg < kth, torch.full_like(lg, -float("inf")), lg)
    pr = torch.softmax(lg, -1)
    if 0.0 < p.top_p < 1.0:
        sp, si = torch.sort(pr, descending=True)
        keep = torch.cumsum(sp, 0) - sp < p.top_p
        mask = torch.zeros_like(pr, dtype=torch.bool)
        mask[si[keep]] = True
        pr = torch.where(mask, pr, torch.zeros_like(pr))
        pr = pr / pr.sum()
    return pr


def sample_from(pr: torch.Tensor, seed: int, pos: int) -> int:
    g = torch.Generator().manual_seed(splitmix64(seed, pos) & 0x7FFFFFFFFFFFFFFF)
    return int(torch.multinomial(pr, 1, generator=g))


class SpecRoundGovernor:
    """EMA of the per-round speculative gain (tokens x plain_ms - round_ms); drafting is suspended
    while the gain is negative and probed again every ``probe_every`` rounds."""

    def __init__(self, alpha: float = 0.2, probe_every: int = 16, enabled: bool = True):
        self.alpha, self.probe_every, self.enabled = alpha, probe_every, enabled
        self.gain_ema = 0.0
        self.rounds = 0
        self.plain_ms = None

    def observe_plain(self, ms: float):
        self.plain_ms = ms if self.plain_ms is None else (1 - self.alpha) * self.plain_ms + self.alpha * ms

    def observe_round(self, tokens: int, round_ms: float):
        if self.plain_ms is None:
            return
        gain = tokens * self.plain_ms - round_ms
        self.gain_ema = (1 - self.alpha) * self.gain_ema + self.alpha * gain

    def should_draft(self) -> bool:
        self.rounds += 1
        if not self.enabled or self.plain_ms is None:
            return True
        return self.gain_ema >= 0 or self.rounds % self.probe_every == 0


class _DegradedRetry(Exception):
    """The prefill of a retry-eligible request ran with an expert missing (a capped expert cache under a fetch deadline finished the
    step without it): the attempt is abandoned before a single token is emitted, so even a streaming request can be run again."""


class Orchestrator:
    """Serves InferenceRequests on one engine.  ``draft`` is an optional proposer with
    ``propose(context_ids, gamma) -> List[int]`` (speculative decoding)."""

    def __init__(self, engine, eos_token_ids: Sequence[int] = (), prefix_cache: Optional[PrefixCacheConfig] = None,
                 draft=None, speculation_depth: int = 0, tokenizer=None, governor: Optional[SpecRoundGovernor] = None, max_batch: int = 1,
                 prefill_slice_tokens: int = 0, degraded_retry_max: int = 0, depth_policy=None, reasoning=None):
        """``max_batch`` > 1: continuous batching - up to that many plain greedy requests decode together, one engine step per token
        of ALL of them; a request joins after its own prefill and leaves when it finishes, the others never wait for it.  Requests
        that need more than the arg-max of a step (sampling on the host, log-probabilities, guided decoding, speculation) are
        served one at a time between batches, in arrival order.  The reference serves one request at a time
        (python/cli/serve.py:273 clamps the batch to 1); this is the serving form of the engine's batched decode step."""
        self.engine = engine
        # a request whose prefill was computed without a router-selected expert (the engine's graceful degradation under a fetch
        # deadline) is a known-wrong answer: run it again up to this many times before delivering it; every action is counted, a retry
        # loop that hides a capacity problem would be worse than the problem (reference: orchestrator.py degraded_retry_max)
        self.degraded_retry_max = max(0, int(degraded_retry_max))
        self.degraded_retries_total = self.degraded_delivered_total = 0
        self.max_batch = max(1, int(max_batch))
        self.running: List[list] = []             # continuous batching: [request, sequence id, next token to feed]
        self.batched_steps = 0
        # continuous batching: a joining request's prompt is prefilled in slices of this many tokens, one slice between two decode
        # steps of the running batch, so the others wait for a slice (tens of milliseconds), not for a whole long prompt (seconds);
        # 0 = four of the engine's prefill chunks
        self.prefill_slice = int(prefill_slice_tokens) or 4 * int(getattr(getattr(engine, "_engine", engine), "prefill_chunk", 0) or 2048)
        # admission back-pressure: a request that could not get KV pages or a sequence slot while others are decoding goes back to the
        # head of the queue and waits until one of them has finished (instead of failing)
        self._admit_hold: Optional[int] = None    # admit again once fewer than this many requests are running
        self.admission_waits = 0
        self.preemptions = 0
        self.joining: Optional[list] = None       # [request, sequence id, prompt, tokens already in the sequence, degraded steps before]
        self.prefill_slices = 0
        self.eos = set(int(t) for t in eos_token_ids)
        self.prefix = PrefixCache(engine, prefix_cache or PrefixCacheConfig())
        self.draft, self.gamma = draft, speculation_depth if draft is not None else 0
        # optional ``speculation.combiner.DepthPolicy``: the depth asked of the draft follows the measured acceptance (0 = a plain step)
        self.depth_policy = depth_policy if draft is not None else None
        # optional (``speculation.policies.ReasoningMode``, think-open ids, think-close ids): inside a think block the depth asked of the
        # draft is multiplied (long, low-entropy reasoning text accepts deeper drafts)
        self.reasoning = reasoning if (draft is not None and reasoning is not None and reasoning[0].enabled) else None
        self._think = None
        self.think_rounds = 0
        self.tokenizer = tokenizer
        self.governor = governor or SpecRoundGovernor(enabled=False)
        self.queue: Deque[InferenceRequest] = collections.deque()
        self.lock = threading.Lock()
        self.wake = threading.Event()
        self.stop_flag = threading.Event()
        self.active: Optional[InferenceRequest] = None
        self.served = 0
        self.gpu_fatal: Optional[str] = None      # set once by the first sticky device error; /health reports it, new work is refused
        # native statistics of the speculation rounds (global / windowed / per-request acceptance, expected tokens per round) and
        # a seqlock-published state block that other threads (the HTTP server's /health) read without taking the serving lock
        from ..runtime import native as _rt
        self.acceptance = _rt.AcceptanceTracker()
        self._state = _rt.StateSnapshot(64)
        self._gen_tokens = 0
        self._publish_state()

    # ---- published state (single writer: the serving thread; any number of readers) ----
    _STATE_FMT = "<qqqqddqq"    # served, queued, generated tokens, free KV pages, acceptance (windowed), wall time of the last update,
                                # requests decoding together right now, batched decode steps so far

    def _publish_state(self):
        import struct
        free_pages = -1
        try:
            free_pages = int(self.engine.free_page_count())
        except Exception:      # engines without a page pool
            pass
        blob = struct.pack(self._STATE_FMT, self.served, len(self.queue), self._gen_tokens, free_pages, float(self.acceptance.windowed_rate()), time.time(),
                           len(getattr(self, "running", ())) + (1 if getattr(self, "joining", None) is not None else 0), getattr(self, "batched_steps", 0))
        self._state.begin(); self._state.write(0, blob); self._state.end()

    def published_state(self) -> dict:
        """A consistent copy of the last published state block (lock-free read; retried while the writer is mid-update)."""
        import struct
        raw, version = self._state.read(0, struct.calcsize(self._STATE_FMT))
        if raw is None:
            return {}
        served, queued, gen, free_pages, acc, t, running, bsteps = struct.unpack(self._STATE_FMT, raw)
        return {"served": served, "queued": queued, "generated_tokens": gen, "free_kv_pages": free_pages, "spec_acceptance_windowed": round(acc, 4),
                "state_age_s": round(max(0.0, time.time() - t), 3), "running": running, "batched_steps": bsteps}

    # ---- thread-safe entry points ----
    def submit_request(self, req: InferenceRequest):
        req.stats.t_submit = time.time()
        if self.gpu_fatal is not None:
            # the device is gone: every step would fail the same way, so the request is refused at once with the recorded cause
            req.error = f"gpu_fatal: {self.gpu_fatal}"
            self._finish(req, "error")
            return
        with self.lock:
            self.queue.append(req)
        self.wake.set()

    def cancel_request(self, request_id: str) -> bool:
        with self.lock:
            for r in list(self.queue):
                if r.request_id == request_id:
                    self.queue.remove(r)
                    self._finish(r, "cancelled")
                    return True
            if self.active is not None and self.active.request_id == request_id:
                self.active.cancelled.set()
                return True
            for r in self.running + ([self.joining] if self.joining is not None else []):
                if r[0].request_id == request_id:
                    r[0].cancelled.set()                  # leaves the batch at its next token (a joining request: after its current slice)
                    return True
        return False

    def queued(self) -> int:
        with self.lock:
            return len(self.queue)

    def shutdown(self):
        self.stop_flag.set()
        self.wake.set()

    # ---- main loop ----
    def run(self, idle_sleep_s: float = 0.0002):
        last_sweep = 0.0
        while not self.stop_flag.is_set():
            if not self.step():
                # nothing to serve: the idle-time tiering of prefix holders (HBM -> pinned host -> file), never on the request path
                now = time.monotonic()
                if now - last_sweep >= 1.0:
                    last_sweep = now
                    try:
                        self.prefix.idle_sweep(now)
                    except Exception as exc:  # noqa: BLE001 - housekeeping must not kill the serving loop
                        self.last_sweep_error = f"{type(exc).__name__}: {exc}"
                self.wake.wait(timeout=0.05)
                self.wake.clear()

    def step(self) -> bool:
        """Serve one queued request to completion (``max_batch`` == 1), or advance the running batch by one token and admit one
        waiting request (continuous batching); False when there is nothing to do."""
        if self.max_batch > 1:
            return self._step_batched()
        with self.lock:
            if not self.queue:
                return False
            req = self.queue.popleft()
            self.active = req
        try:
            while True:
                try:
                    self._generate(req)
                    break
                except _DegradedRetry:
                    req.stats.degraded_retries += 1
                    self.degraded_retries_total += 1
        except Exception as exc:  # noqa: BLE001 - a failed request must not kill the serving loop
            req.error = f"{type(exc).__name__}: {exc}"
            if is_gpu_fatal(exc) and self.gpu_fatal is None:
                # a sticky device error (illegal access, launch failure, lost device): recorded ONCE, reported by /health, and every
                # queued or later request is failed with it instead of being run into the same wall
                self.gpu_fatal = req.error[:300]
                log.error("GPU fatal error, serving stops accepting work: %s", self.gpu_fatal)
                with self.lock:
                    waiting, self.queue = list(self.queue), collections.deque()
                for r in waiting:
                    r.error = f"gpu_fatal: {self.gpu_fatal}"
                    self._finish(r, "error")
            self._finish(req, "error")
        finally:
            with self.lock:
                self.active = None
            self.served += 1
        return True

    # ---- continuous batching ----
    def _batchable(self, req: InferenceRequest) -> bool:
        p = req.params
        return p.greedy and p.logprobs == 0 and req.logit_mask is None and self.gamma == 0

    def _fail(self, req: InferenceRequest, exc: BaseException):
        req.error = f"{type(exc).__name__}: {exc}"
        if is_gpu_fatal(exc) and self.gpu_fatal is None:
            self.gpu_fatal = req.error[:300]
            log.error("GPU fatal error, serving stops accepting work: %s", self.gpu_fatal)
            with self.lock:
                waiting, self.queue = list(self.queue), collections.deque()
            for r in waiting:
                r.error = f"gpu_fatal: {self.gpu_fatal}"
                self._finish(r, "error")
        self._finish(req, "error")
        self.served += 1

    def _step_batched(self) -> bool:
        eng = self.engine
        did = False
        # 1. admission: one request joins at a time; its prompt is prefilled slice by slice, one slice per iteration
        if self._admit_hold is not None and len(self.running) < self._admit_hold:
            self._admit_hold = None                        # somebody finished: try again
        if self.joining is None and self._admit_hold is None:
            with self.lock:
                head = self.queue[0] if self.queue else None
                take = head is not None and ((self._batchable(head) and len(self.running) < self.max_batch) or (not self._batchable(head) and not self.running))
                if take:
                    self.queue.popleft()
            if take:
                did = True
                if not self._batchable(head):
                    # needs its own decode arm: served alone, to completion, while no batch is running (arrival order is kept)
                    self.active = head
                    try:
                        self._generate(head)
                    except Exception as exc:  # noqa: BLE001
                        self._fail(head, exc)
                    else:
                        self.served += 1
                    finally:
                        self.active = None
                else:
                    try:
                        self.joining = self._begin(head)
                    except Exception as exc:  # noqa: BLE001
                        if self.running and self._is_capacity_error(exc):
                            self._wait_for_capacity(head)
                        else:
                            self._fail(head, exc)
        if self.joining is not None:
            did = True
            req, sid, prompt, _, d0 = self.joining
            try:
                done_prefill, tok = self._prefill_slice(self.joining)
                if req.cancelled.is_set():
                    eng.free_sequence(sid)
                    self._finish(req, "cancelled")
                    self.served += 1
                    self.joining = None
                elif done_prefill:
                    self.joining = None
                    degraded = self._degraded_count() - d0
                    if degraded > 0:                       # KV rows computed with an expert missing are never cached
                        req.stats.moe_degraded_steps += degraded
                        self.degraded_delivered_total += 1
                    else:
                        self.prefix.register(sid, prompt)
                    if self._emit(req, tok, None):
                        eng.free_sequence(sid)
                        self._finish(req, req.finish_reason or "cancelled")
                        self.served += 1
                    else:
                        self.running.append([req, sid, tok])
            except Exception as exc:  # noqa: BLE001
                self.joining = None
                if sid in getattr(eng, "seqs", {sid: None}):
                    try:
                        eng.free_sequence(sid)
                    except Exception:  # noqa: BLE001
                        pass
                if self.running and self._is_capacity_error(exc):
                    self._wait_for_capacity(req)          # nothing was emitted during the join: the prompt is simply fed again later
                else:
                    self._fail(req, exc)
        # 2. one token for every running request
        if self.running:
            did = True
            sids, toks = [r[1] for r in self.running], [r[2] for r in self.running]
            try:
                outs = self._with_pool_evict_retry(self.running[0][0], lambda: eng.decode(sids, toks))
            except Exception as exc:  # noqa: BLE001 - the step failed for the whole batch
                if len(self.running) > 1 and self._is_capacity_error(exc):
                    # out of KV pages in mid-decode: the youngest request gives its pages back and joins again later, its prompt
                    # and the tokens it has produced fed as one prompt (greedy decoding: the continuation is the same); the step
                    # is run again for the others
                    req, sid, _ = self.running.pop()
                    eng.free_sequence(sid)
                    req.stats.preemptions += 1
                    self.preemptions += 1
                    self._wait_for_capacity(req)
                    return True
                for req, sid, _ in self.running:
                    eng.free_sequence(sid)
                    self._fail(req, exc)
                self.running = []
                return True
            self.batched_steps += 1
            keep = []
            for entry, tok in zip(self.running, outs):
                req, sid, _ = entry
                if self._emit(req, int(tok), None):
                    eng.free_sequence(sid)
                    self._finish(req, req.finish_reason or ("cancelled" if req.cancelled.is_set() else "stop"))
                    self.served += 1
                else:
                    entry[2] = int(tok)
                    keep.append(entry)
            self.running = keep
        return did

    @staticmethod
    def _is_capacity_error(exc: BaseException) -> bool:
        return isinstance(exc, KvPoolExhausted) or "no free sequence slot" in str(exc)

    def _wait_for_capacity(self, req: InferenceRequest):
        with self.lock:
            self.queue.appendleft(req)
        self._admit_hold = len(self.running)
        self.admission_waits += 1

    def _begin(self, req: InferenceRequest) -> list:
        """Prefix lookup and sequence of a joining greedy request: [request, sequence id, prompt, tokens already in the sequence]."""
        eng, st = self.engine, req.stats
        st.t_start = st.t_start or time.time()
        st.prompt_tokens = len(req.prompt_ids)
        if not req.prompt_ids:
            raise ValueError("empty prompt")
        prompt = list(req.prompt_ids) + list(req.output_ids)      # a preempted request resumes behind what it has produced
        sid, cached = self.prefix.fork_from(prompt)
        if sid is None:
            sid = self._with_pool_evict_retry(req, eng.create_sequence)
            cached = 0
        st.cached_tokens = cached
        return [req, sid, prompt, max(cached, eng.seq_len(sid)), self._degraded_count()]

    def _prefill_slice(self, joining: list):
        """Feed the next slice of the joining request's prompt: (prompt complete, the engine's next token after the slice)."""
        req, sid, prompt, fed = joining[:4]
        n = min(self.prefill_slice, len(prompt) - fed)
        tok = self._with_pool_evict_retry(req, lambda: self.engine.prefill(sid, prompt[fed: fed + n]))
        joining[3] = fed + n
        self.prefill_slices += 1
        return joining[3] >= len(prompt), tok

    def _finish(self, req: InferenceRequest, reason: str):
        req.finish_reason = req.finish_reason or reason
        req.stats.t_done = time.time()
        req.stats.completion_tokens = len(req.output_ids)
        self._gen_tokens += len(req.output_ids)
        self.acceptance.forget(hash(req.request_id) & 0x7FFFFFFF)
        self._publish_state()
        req.done.set()
        if req.on_done:
            req.on_done(req)

    def _with_pool_evict_retry(self, req: InferenceRequest, fn):
        """Run ``fn``; on KV pool exhaustion evict one prefix holder and retry the identical step."""
        while True:
            try:
                return fn()
            except KvPoolExhausted:
                if not self.prefix.evict_one():
                    raise
                req.stats.pool_evict_retries += 1

    # ---- one request ----
    def _emit(self, req: InferenceRequest, tok: int, logits: Optional[torch.Tensor]) -> bool:
        """Append a token; returns True when generation must stop."""
        p = req.params
        if not req.output_ids:
            req.stats.t_first_token = time.time()
        req.output_ids.append(tok)
        if self._think is not None:
            self._think.feed(tok)
        info = None
        if p.logprobs and logits is not None:
            lp = torch.log_softmax(logits.float(), -1)
            top = torch.topk(lp, min(p.logprobs, lp.numel()))
            info = {"logprob": float(lp[tok]), "top": [(int(i), float(v)) for v, i in zip(top.values, top.indices)]}
        if req.on_token:
            req.on_token(tok, info)
        if (not p.ignore_eos and tok in self.eos) or tok in p.stop_token_ids:
            req.finish_reason = "stop"
            return True
        if p.stop and self.tokenizer is not None:
            text = self.tokenizer.decode(req.output_ids[-32:])
            if any(s and s in text for s in p.stop):
                req.finish_reason = "stop"
                return True
        if len(req.output_ids) >= p.max_tokens:
            req.finish_reason = "length"
            return True
        return req.cancelled.is_set()

    def _pick(self, req: InferenceRequest, logits: torch.Tensor, pos: int) -> int:
        p = req.params
        if req.logit_mask is not None:
            mask = req.logit_mask(req.output_ids)
            if mask is not None:
                logits = torch.where(mask, logits, torch.full_like(logits, -float("inf")))
        if p.greedy:
            return int(torch.argmax(logits))
        return sample_from(target_probs(logits, p), p.seed if p.seed is not None else 0, pos)

    def _generate(self, req: InferenceRequest):
        eng, p = self.engine, req.params
        st = req.stats
        st.t_start = time.time()
        st.prompt_tokens = len(req.prompt_ids)
        prompt = list(req.prompt_ids)
        if not prompt:
            raise ValueError("empty prompt")
        sid, cached = self.prefix.fork_from(prompt)
        if sid is None:
            sid = self._with_pool_evict_retry(req, eng.create_sequence)
            cached = 0
        st.cached_tokens = cached
        # sampled requests without a logit mask or logprobs draw on the device when the engine can (4 bytes per token come back
        # instead of the vocabulary's logits)
        dev_sample = (not p.greedy) and p.logprobs == 0 and req.logit_mask is None and getattr(eng, "supports_device_sampling", False)
        need_logits = ((not p.greedy) and not dev_sample) or p.logprobs > 0 or req.logit_mask is not None
        try:
            # every attempt feeds what is still missing (the engine's prefill reserves its pages up front and fails before it
            # commits anything, and even an engine that failed mid-prompt is continued, never re-fed)
            d0 = self._degraded_count()
            out = self._with_pool_evict_retry(req, lambda: eng.prefill(sid, prompt[max(cached, eng.seq_len(sid)):], want_logits=need_logits))
            degraded = self._degraded_count() - d0
            if degraded > 0:
                # the KV rows of this prefill were computed with an expert missing: never cached, and the attempt is run again while
                # the request has retry budget (nothing has been emitted yet)
                if req.stats.degraded_retries < self.degraded_retry_max:
                    raise _DegradedRetry()
                req.stats.moe_degraded_steps += degraded
                self.degraded_delivered_total += 1
            else:
                self.prefix.register(sid, prompt)
            tok, logits = out if need_logits else (out, None)
            if need_logits:
                tok = self._pick(req, logits, len(prompt))
            elif dev_sample:
                # the prompt's last position: rewind one token and let the sampled decode step produce the first token
                tok = self._first_sampled_token(req, sid, prompt)
            if self._emit(req, tok, logits):
                return self._finish(req, req.finish_reason or "cancelled")
            if dev_sample:
                self._decode_plain(req, sid, tok, False, sample=self._sample_args(req))
            elif self.gamma > 0 and not need_logits:
                self._begin_speculation(req)
                self._decode_speculative(req, sid, tok)
            elif self.gamma > 0 and not getattr(eng, "has_recurrent_state", False):
                self._begin_speculation(req)
                self._decode_speculative_logits(req, sid, tok)
            else:
                self._decode_plain(req, sid, tok, need_logits)
            self._finish(req, req.finish_reason or ("cancelled" if req.cancelled.is_set() else "stop"))
        finally:
            self._think = None
            eng.free_sequence(sid)

    def _degraded_count(self) -> int:
        """Degraded steps the engine has run so far (a capped expert cache that finished steps without a late expert), else 0."""
        eng = getattr(self.engine, "_engine", self.engine)
        st = getattr(getattr(eng, "model", None), "streamer", None)
        if st is not None:
            return int(st.stats.get("degraded_steps", 0))
        return int(getattr(eng, "degraded_steps", 0) or 0)

    def _sample_args(self, req: InferenceRequest):
        p = req.params
        return (p.temperature, p.top_k, p.top_p, p.seed if p.seed is not None else 0)

    def _first_sampled_token(self, req: InferenceRequest, sid: int, prompt: List[int]) -> int:
        """Device-sampled requests: the prefill returned the greedy token of the last prompt position; the sampled one is drawn
        from that position's logits, which are still in the engine's prefill workspace."""
        eng = self.engine
        return eng.sample_last_prefill(sid, self._sample_args(req))

    def _decode_plain(self, req: InferenceRequest, sid: int, tok: int, need_logits: bool, sample=None):
        eng = self.engine
        while True:
            t0 = time.time()
            if sample is not None:
                tok = self._with_pool_evict_retry(req, lambda: eng.decode([sid], [tok], sample=sample))[0]
                logits = None
            elif need_logits:
                outs, lg = self._with_pool_evict_retry(req, lambda: eng.decode([sid], [tok], return_logits=True))
                logits = lg[0]
                tok = self._pick(req, logits, len(req.prompt_ids) + len(req.output_ids))
            else:
                tok = self._with_pool_evict_retry(req, lambda: eng.decode([sid], [tok]))[0]
                logits = None
            self.governor.observe_plain((time.time() - t0) * 1e3)
            if self._emit(req, tok, logits):
                return

    def _decode_speculative_logits(self, req: InferenceRequest, sid: int, tok: int):
        """Lossless speculation for requests that need the logits of every step (sampling, guided decoding, logprobs).
        The draft is a point mass, so exact rejection sampling reduces to equality coupling: draw s_k from the target
        distribution of row k (temperature / top-k / top-p / mask applied, RNG keyed by the absolute position) and accept
        the draft token iff s_k equals it; on a mismatch s_k itself is the correct next token.  One RNG draw per committed
        token at its own position => the same trajectory as plain sampled decoding for a fixed seed.
        Reference behaviour: python/orchestrator/orchestrator.py:3781-3818 (_decode_speculative_sampled), guided variant
        :4079-4237."""
        eng = self.engine
        while True:
            t0 = time.time()
            gamma = self._round_depth()
            if gamma <= 0 or not self.governor.should_draft():
                lg = self._with_pool_evict_retry(req, lambda: eng.decode([sid], [tok], return_logits=True))[1][0]
                tok = self._pick(req, lg, len(req.prompt_ids) + len(req.output_ids))
                self.governor.observe_plain((time.time() - t0) * 1e3)
                if self._emit(req, tok, lg):
                    return
                continue
            ctx = list(req.prompt_ids) + req.output_ids
            draft = list(self.draft.propose(ctx, gamma))[:gamma]
            base_len = eng.seq_len(sid)
            rows = [tok] + draft
            logits = self._with_pool_evict_retry(req, lambda: eng.forward_rows(sid, rows, commit=True))
            n_acc, n_new, stop = 0, 0, False
            for k in range(len(rows)):
                t = self._pick(req, logits[k], len(req.prompt_ids) + len(req.output_ids))
                n_new += 1
                tok = t
                if self._emit(req, t, logits[k]):
                    stop = True
                    break
                if k < len(draft) and t == draft[k]:
                    n_acc += 1
                    continue
                break
            eng.rewind(sid, base_len + 1 + n_acc)
            req.stats.spec_rounds += 1
            req.stats.spec_accepted += n_acc
            self.acceptance.record(hash(req.request_id) & 0x7FFFFFFF, len(draft), n_acc)
            self.governor.observe_round(n_new, (time.time() - t0) * 1e3)
            if hasattr(self.draft, "feedback"):
                self.draft.feedback(len(draft), n_acc)
            if self.depth_policy is not None:
                self.depth_policy.record(len(draft), n_acc)
            if stop:
                return

    def _round_depth(self) -> int:
        d = self.gamma if self.depth_policy is None else min(self.gamma, self.depth_policy.depth())
        if self._think is not None and self._think.thinking and d > 0:
            mode = self.reasoning[0]
            d = max(d, mode.depth(d, mode.overrides(True)))
            self.think_rounds += 1
        return d

    def _begin_speculation(self, req: InferenceRequest):
        if self.depth_policy is not None:
            self.depth_policy.begin_request()
        self._think = None
        if self.reasoning is not None:
            from ..speculation.policies import ThinkTracker
            self._think = ThinkTracker(self.reasoning[1], self.reasoning[2])
            for t in list(req.prompt_ids)[-4096:] + list(req.output_ids):     # a prompt may end inside an open think block
                self._think.feed(int(t))

    def _decode_speculative(self, req: InferenceRequest, sid: int, tok: int):
        """Greedy lossless speculation: the draft proposes up to gamma tokens after ``tok``; one batched
        target forward over [tok, d_0..d_{g-1}] gives the target's argmax at every position; the longest
        agreeing prefix is accepted plus the target's own next token (correction or bonus)."""
        eng = self.engine
        dev_verify = hasattr(eng, "verify_greedy")            # decides on the device, rolls recurrent state back through anchors
        recurrent = getattr(eng, "has_recurrent_state", False) and not dev_verify
        while True:
            gamma = self._round_depth()
            if recurrent or gamma <= 0 or not self.governor.should_draft():
                t0 = time.time()
                tok = self._with_pool_evict_retry(req, lambda: eng.decode([sid], [tok]))[0]
                self.governor.observe_plain((time.time() - t0) * 1e3)
                if self._emit(req, tok, None):
                    return
                continue
            t0 = time.time()
            ctx = list(req.prompt_ids) + req.output_ids
            draft = list(self.draft.propose(ctx, gamma))[:gamma]
            base_len = eng.seq_len(sid)
            rows = [tok] + draft
            if dev_verify:
                n_acc, nxt = self._with_pool_evict_retry(req, lambda: eng.verify_greedy(sid, tok, draft))
            else:
                logits = self._with_pool_evict_retry(req, lambda: eng.forward_rows(sid, rows, commit=True))
                target = [int(t) for t in torch.argmax(logits, -1)]
                n_acc = 0
                while n_acc < len(draft) and draft[n_acc] == target[n_acc]:
                    n_acc += 1
                nxt = target[n_acc]
                eng.rewind(sid, base_len + 1 + n_acc)          # keep tok + the accepted draft tokens
            req.stats.spec_rounds += 1
            req.stats.spec_accepted += n_acc
            self.acceptance.record(hash(req.request_id) & 0x7FFFFFFF, len(draft), n_acc)
            new = draft[:n_acc] + [nxt]
            self.governor.observe_round(len(new), (time.time() - t0) * 1e3)
            if hasattr(self.draft, "feedback"):
                self.draft.feedback(len(draft), n_acc)
            if self.depth_policy is not None:
                self.depth_policy.record(len(draft), n_acc)
            for t in new:
                if self._emit(req, t, None):
                    return
            tok = new[-1]
