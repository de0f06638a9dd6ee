"""Serving stack on the CPU null engine: orchestrator arms, prefix cache, parsers, guided JSON, HTTP API."""
import json
import threading

import pytest
import torch

from layerstorm_b200 import build as _build

_build.build_all(only="runtime")

from layerstorm_b200.runtime.null_engine import NullEngine
from layerstorm_b200.serving.guided import JsonPrefixValidator, make_logit_mask
from layerstorm_b200.serving.orchestrator import InferenceRequest, Orchestrator, SamplingParams
from layerstorm_b200.serving.parsers import (StreamingReasoningSplitter, get_reasoning_parser, get_tool_parser)
from layerstorm_b200.serving.prefix_cache import PrefixCacheConfig
from layerstorm_b200.serving.tokenizer import ChatTemplateRenderer, IncrementalDetokenizer, TokenizerWrapper


def run(orch, prompt, **kw):
    req = InferenceRequest("r", list(prompt), SamplingParams(**kw))
    orch.submit_request(req)
    assert orch.step()
    assert req.done.is_set() and req.error is None, req.error
    return req


def test_greedy_matches_plain_loop_and_prefix_cache_is_invisible():
    prompt = list(range(5, 205))
    ref_eng = NullEngine()
    sid = ref_eng.create_sequence()
    t = ref_eng.prefill(sid, prompt)
    ref = [t]
    for _ in range(15):
        t = ref_eng.decode([sid], [t])[0]
        ref.append(t)
    for cache in (False, True):
        eng = NullEngine()
        orch = Orchestrator(eng, prefix_cache=PrefixCacheConfig(enabled=cache, grid=64, min_prefix=64))
        r1 = run(orch, prompt, max_tokens=16, ignore_eos=True)
        r2 = run(orch, prompt[:150] + [9, 9, 9], max_tokens=4, ignore_eos=True)
        r3 = run(orch, prompt, max_tokens=16, ignore_eos=True)
        assert r1.output_ids == ref and r3.output_ids == ref
        if cache:
            assert r3.stats.cached_tokens == 192 and r2.stats.cached_tokens == 128
            assert eng.prefill_tokens == 200 + (153 - 128) + (200 - 192)
        else:
            assert r3.stats.cached_tokens == 0
    # every sequence is released (holders stay): free slots + holders == max_seqs
    assert len(eng.free_slots) + orch.prefix.holders() == eng.max_seqs


def test_speculative_is_lossless_and_pool_evict_retry():
    prompt = list(range(3, 90))

    class GoodThenBadDraft:
        def __init__(self, eng): self.eng = eng
        def propose(self, ctx, gamma):
            out, c = [], list(ctx)
            for i in range(gamma):
                t = self.eng._next(c) if i < 3 else 7      # three right, then wrong
                out.append(t); c.append(t)
            return out

    plain = run(Orchestrator(NullEngine()), prompt, max_tokens=24, ignore_eos=True).output_ids
    eng = NullEngine()
    orch = Orchestrator(eng, draft=GoodThenBadDraft(eng), speculation_depth=6)
    r = run(orch, prompt, max_tokens=24, ignore_eos=True)
    assert r.output_ids == plain
    assert r.stats.spec_rounds > 0 and r.stats.spec_accepted >= 3 * (r.stats.spec_rounds - 1)
    # KV pool too small for a holder + a new request: the holder is evicted and the step retried
    eng = NullEngine(max_seqs=4, max_ctx=256, page=16, num_pages=12)
    orch = Orchestrator(eng, prefix_cache=PrefixCacheConfig(grid=16, min_prefix=16))
    run(orch, list(range(100, 200)), max_tokens=2, ignore_eos=True)
    r = run(orch, list(range(300, 420)), max_tokens=2, ignore_eos=True)
    assert r.stats.pool_evict_retries >= 1 and r.finish_reason == "length"


def test_sampling_is_seeded_and_cancel():
    orch = Orchestrator(NullEngine())
    a = run(orch, [1, 2, 3], max_tokens=8, temperature=1.0, top_k=20, top_p=0.9, seed=11, ignore_eos=True)
    b = run(orch, [1, 2, 3], max_tokens=8, temperature=1.0, top_k=20, top_p=0.9, seed=11, ignore_eos=True)
    c = run(orch, [1, 2, 3], max_tokens=8, temperature=1.0, top_k=20, top_p=0.9, seed=12, ignore_eos=True)
    assert a.output_ids == b.output_ids and a.output_ids != c.output_ids
    req = InferenceRequest("x", [1, 2], SamplingParams(max_tokens=1000, ignore_eos=True))
    req.on_token = lambda t, i: req.cancelled.set() if len(req.output_ids) >= 5 else None
    orch.submit_request(req); orch.step()
    assert req.finish_reason == "cancelled" and len(req.output_ids) == 5
    q = InferenceRequest("q", [1], SamplingParams())
    orch.submit_request(q)
    assert orch.cancel_request("q") and q.finish_reason == "cancelled" and not orch.step()


def test_parsers():
    text = "I will call.<tool_call>get_weather\n<arg_key>city</arg_key>\n<arg_value>Paris</arg_value>\n<arg_key>days</arg_key>\n<arg_value>3</arg_value>\n</tool_call>"
    rest, calls = get_tool_parser("glm47").parse(text)
    assert rest == "I will call." and calls[0].name == "get_weather" and json.loads(calls[0].arguments) == {"city": "Paris", "days": 3}
    ds = '<｜tool▁calls▁begin｜><｜tool▁call▁begin｜>search<｜tool▁sep｜>{"q": "b200"}<｜tool▁call▁end｜><｜tool▁calls▁end｜>'
    rest, calls = get_tool_parser("deepseek_v4").parse(ds)
    assert rest == "" and calls[0].name == "search" and json.loads(calls[0].arguments) == {"q": "b200"}
    rp = get_reasoning_parser("glm45")
    assert rp.parse("<think>hmm</think>\nanswer") == ("hmm", "answer") and rp.parse("plain") == (None, "plain")
    sp = StreamingReasoningSplitter(rp)
    r_all, c_all = "", ""
    for piece in ["<th", "ink>rea", "son</thi", "nk>\nfi", "nal"]:
        r, c = sp.push(piece); r_all += r; c_all += c
    assert (r_all, c_all) == ("reason", "final")
    with pytest.raises(ValueError):
        get_tool_parser("nope")


def test_guided_json_and_detokenizer():
    v = JsonPrefixValidator()
    assert v.feed_text('{"a": [1, 2.5e3, true, null, {"b": "x\\n"}], "c": {}}') and v.complete
    for bad in ['{"a" 1}', '[1]', '{"a": 01}', '{,}', '{"a": tru }']:
        assert not JsonPrefixValidator().feed_text(bad), bad
    tok = TokenizerWrapper()
    mask = make_logit_mask(tok, {"type": "json_object"})
    eng = NullEngine(vocab=tok.vocab_size)
    orch = Orchestrator(eng, eos_token_ids=tok.eos_token_ids, tokenizer=tok)
    req = InferenceRequest("g", tok.encode("give json"), SamplingParams(max_tokens=200), logit_mask=mask)
    orch.submit_request(req); orch.step()
    out = tok.decode(req.output_ids)
    vv = JsonPrefixValidator()
    assert vv.feed_text(out)                      # always a valid JSON prefix
    if req.finish_reason == "stop":
        json.loads(out)
    d = IncrementalDetokenizer(tok)
    s = "".join(d.push(t) for t in tok.encode("héllo ✓ wörld"))
    assert s == "héllo ✓ wörld"
    assert "user" in ChatTemplateRenderer().render([{"role": "user", "content": "hi"}])


def test_http_api():
    from fastapi.testclient import TestClient
    from layerstorm_b200.serving.http_server import LayerStormServer, ServerConfig
    tok = TokenizerWrapper()
    eng = NullEngine(vocab=tok.vocab_size)
    orch = Orchestrator(eng, eos_token_ids=tok.eos_token_ids, tokenizer=tok)
    th = threading.Thread(target=orch.run, daemon=True)
    th.start()
    srv = LayerStormServer(orch, tok, ServerConfig(model_name="m", max_queued_requests=2, reasoning_parser="glm45"))
    c = TestClient(srv.app)
    assert c.get("/health").json()["status"] == "ok"
    assert c.get("/v1/models").json()["data"][0]["id"] == "m"
    r = c.post("/v1/completions", json={"prompt": "hello", "max_tokens": 5, "ignore_eos": True, "logprobs": 2}).json()
    assert r["usage"]["completion_tokens"] == 5 and r["choices"][0]["finish_reason"] == "length"
    assert len(r["choices"][0]["logprobs"]["content"]) == 5
    r = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "hi"}], "max_tokens": 6, "ignore_eos": True}).json()
    assert r["choices"][0]["message"]["role"] == "assistant" and r["usage"]["completion_tokens"] == 6
    with c.stream("POST", "/v1/chat/completions", json={"messages": [{"role": "user", "content": "hi"}], "max_tokens": 6, "stream": True, "ignore_eos": True}) as s:
        lines = [l for l in s.iter_lines() if l.startswith("data: ")]
    assert lines[-1] == "data: [DONE]" and json.loads(lines[-2][6:])["choices"][0]["finish_reason"] == "length"
    assert c.post("/v1/completions", json={"prompt": 5}).status_code == 400
    assert c.post("/v1/chat/completions", json={"messages": []}).status_code == 400
    srv.inflight = 3
    r = c.post("/v1/completions", json={"prompt": "x"})
    assert r.status_code == 503 and "Retry-After" in r.headers
    srv.failed_ranks = lambda: {}                                  # multi-process server: every rank alive
    assert c.get("/health").status_code == 200
    srv.failed_ranks = lambda: {3: "sent no heartbeat for 12.0 s"}
    r = c.get("/health")
    assert r.status_code == 503 and "3: sent no heartbeat" in r.json()["error"]["message"]
    orch.shutdown()


def test_sampled_and_guided_speculation_follow_the_plain_trajectory():
    """Equality coupling: with a fixed seed, speculative sampled decoding emits exactly the tokens of plain sampled decoding,
    whatever the draft proposes; a logit mask (guided decoding) composes with it."""
    from layerstorm_b200.speculation import EngineDraft, PromptLookupDraft
    prompt = [5, 6, 7, 8, 5, 6, 7, 8, 5, 6]

    def run(draft, gamma, mask=None, **sp):
        eng = NullEngine(vocab=64, page=16)
        o = Orchestrator(eng, draft=draft, speculation_depth=gamma)
        req = InferenceRequest("r", list(prompt), SamplingParams(max_tokens=24, ignore_eos=True, **sp))
        req.logit_mask = mask
        o.submit_request(req); o.step()
        return req

    plain = run(None, 0, temperature=0.9, top_k=20, seed=1234)
    good = run(EngineDraft(NullEngine(vocab=64, page=16), 4), 4, temperature=0.9, top_k=20, seed=1234)
    lookup = run(PromptLookupDraft(2, 4, 4), 4, temperature=0.9, top_k=20, seed=1234)
    assert good.output_ids == plain.output_ids == lookup.output_ids
    assert good.stats.spec_rounds > 0 and lookup.stats.spec_rounds > 0
    other = run(None, 0, temperature=0.9, top_k=20, seed=99)
    assert other.output_ids != plain.output_ids                 # the seed matters, i.e. the requests really sample
    even = torch.arange(64) % 2 == 0
    mask = lambda out: even                                      # guided: only even token ids are legal
    g_plain = run(None, 0, mask=mask, temperature=0.7, seed=7)
    g_spec = run(EngineDraft(NullEngine(vocab=64, page=16), 3), 3, mask=mask, temperature=0.7, seed=7)
    assert g_spec.output_ids == g_plain.output_ids and all(t % 2 == 0 for t in g_spec.output_ids)
    lp = run(EngineDraft(NullEngine(vocab=64, page=16), 3), 3, logprobs=2)      # greedy + logprobs also takes the logits path
    assert lp.output_ids == run(None, 0, logprobs=2).output_ids


def test_randomised_requests_with_shared_prefixes_under_pool_pressure():
    """Many requests with overlapping prefixes through a small KV pool: every output equals the plain run of the same prompt, and no
    sequence slot or page leaks however the prefix cache forked, evicted and retried."""
    import random
    rng = random.Random(7)
    stems = [[rng.randrange(4, 500) for _ in range(rng.randrange(40, 120))] for _ in range(4)]
    eng = NullEngine(max_seqs=6, max_ctx=256, page=16, num_pages=40)
    orch = Orchestrator(eng, prefix_cache=PrefixCacheConfig(grid=16, min_prefix=16, max_holders=3))
    total_pages = eng.free_page_count()
    cached = retries = 0
    for n in range(40):
        stem = rng.choice(stems)
        prompt = stem[: rng.randrange(20, len(stem) + 1)] + [rng.randrange(4, 500) for _ in range(rng.randrange(0, 30))]
        gen = rng.randrange(1, 12)
        want = run(Orchestrator(NullEngine(max_ctx=256)), prompt, max_tokens=gen, ignore_eos=True).output_ids
        r = run(orch, prompt, max_tokens=gen, ignore_eos=True)
        assert r.output_ids == want, n
        cached += r.stats.cached_tokens
        retries += r.stats.pool_evict_retries
        assert len(eng.free_slots) + orch.prefix.holders() == eng.max_seqs
    assert cached > 0                                             # the shared stems were reused
    orch.prefix.clear()
    assert len(eng.free_slots) == eng.max_seqs and eng.free_page_count() == total_pages


def test_pool_exhaustion_in_the_middle_of_a_chunked_prefill_does_not_duplicate_the_prefix():
    """An engine whose prefill commits chunk by chunk and runs out of pages at a later chunk: the orchestrator evicts a prefix
    holder and continues from the committed frontier - it must not feed the committed chunks a second time."""
    from layerstorm_b200.runtime.native import KvPoolExhausted

    class ChunkedEngine(NullEngine):
        chunk = 32
        failures = 0

        def prefill(self, sid, tokens, want_logits=False):
            tokens = [int(t) for t in tokens]
            out = None
            for c0 in range(0, len(tokens), self.chunk):
                try:
                    out = NullEngine.prefill(self, sid, tokens[c0: c0 + self.chunk], want_logits)
                except KvPoolExhausted:
                    ChunkedEngine.failures += 1
                    raise
            return out

    prompt_a, prompt_b = list(range(10, 138)), list(range(300, 460))
    ref_eng = NullEngine()
    sid = ref_eng.create_sequence()
    t = ref_eng.prefill(sid, prompt_b)
    ref = [t]
    for _ in range(7):
        t = ref_eng.decode([sid], [t])[0]
        ref.append(t)
    # 14 pages of 16 tokens: request A (128 tokens + 8 generated) leaves a holder of 8 pages; request B needs 11 pages, so its
    # prefill runs out of pages after a few chunks, the holder is evicted and the prefill goes on
    eng = ChunkedEngine(max_seqs=4, max_ctx=512, page=16, num_pages=14)
    orch = Orchestrator(eng, prefix_cache=PrefixCacheConfig(enabled=True, grid=64, min_prefix=64))
    run(orch, prompt_a, max_tokens=8, ignore_eos=True)
    assert orch.prefix.holders() >= 1
    rb = run(orch, prompt_b, max_tokens=8, ignore_eos=True)
    assert ChunkedEngine.failures >= 1, "the scenario must exhaust the pool in the middle of the prompt"
    assert rb.output_ids == ref


def test_device_error_words_raise_a_typed_error():
    from layerstorm_b200.runtime.engine import DeviceWaitError, raise_on_error_words
    raise_on_error_words(["tensor_core", "tp_allreduce"], [0, 0])
    with pytest.raises(DeviceWaitError) as ei:
        raise_on_error_words(["tensor_core", "tp_allreduce"], [0, 103])
    assert ei.value.source == "tp_allreduce" and ei.value.code == 103 and "rank 3" in str(ei.value)


def test_published_state_and_acceptance_statistics():
    """The serving thread publishes a seqlock state block (read lock-free by /health) and feeds the native acceptance tracker."""
    eng = NullEngine()

    class RightDraft:
        def propose(self, ctx, gamma):
            out, c = [], list(ctx)
            for _ in range(gamma):
                c.append(eng._next(c)); out.append(c[-1])
            return out

    orch = Orchestrator(eng, draft=RightDraft(), speculation_depth=3)
    assert orch.published_state()["served"] == 0
    r = run(orch, list(range(5, 60)), max_tokens=12, ignore_eos=True)
    st = orch.published_state()
    assert st["generated_tokens"] == len(r.output_ids) == 12 and st["free_kv_pages"] > 0 and st["state_age_s"] < 60
    assert r.stats.spec_rounds > 0 and orch.acceptance.global_rate() > 0.9 and st["spec_acceptance_windowed"] > 0.9
    assert orch.acceptance.expected_tokens(3) > 3.0


def test_idle_prefix_holders_hibernate_then_spill_under_a_byte_cap_and_a_lost_file_is_a_miss(tmp_path):
    """The idle-time tiering policy of the prefix cache on a fake tiered engine: first hop after ``hibernate_idle_seconds``, second
    hop (leaf holders only, LRU first, one per sweep) after ``spill.idle_seconds``, the byte cap enforced before the write by
    dropping the LRU spilled holder, stale files reclaimed at start-up, a hit on a spilled holder brings it back, a lost file
    degrades to a miss."""
    import os
    import torch
    from layerstorm_b200.runtime.null_engine import NullEngine
    from layerstorm_b200.serving.prefix_cache import PrefixCache, PrefixCacheConfig, PrefixSpillConfig

    class Tiered(NullEngine):
        def __init__(self, **kw):
            super().__init__(**kw)
            self.hibernated, self.spilled = {}, {}
            self.cold_kv = {0: torch.zeros(1, 16, 19200, dtype=torch.uint8)}          # 300 KiB per page
            self.cold_idx = {}

        def hibernate(self, sid):
            self.hibernated[sid] = list(range((self.seqs[sid].length + self.page - 1) // self.page))
            return len(self.hibernated[sid])

        def spill(self, sid, path):
            n = len(self.hibernated.pop(sid)) * 16 * 19200
            open(path, "wb").write(b"x")
            self.spilled[sid] = (path, n)
            return n

        def fork_sequence(self, parent, prefix_len=None):
            if parent in self.spilled:
                open(self.spilled[parent][0], "rb").close()                             # OSError when the file is gone
                self.spilled.pop(parent)
            self.hibernated.pop(parent, None)
            return super().fork_sequence(parent, prefix_len)

        def free_sequence(self, sid):
            if sid in self.spilled:
                path = self.spilled.pop(sid)[0]
                if os.path.exists(path):
                    os.remove(path)
            self.hibernated.pop(sid, None)
            super().free_sequence(sid)

    d = tmp_path / "spill"
    d.mkdir()
    (d / "ls-spill-999-1-1.kvspill").write_bytes(b"stale")
    (d / "keep.txt").write_bytes(b"not ours")
    eng = Tiered(max_seqs=16, max_ctx=512, page=16)
    cfg = PrefixCacheConfig(grid=64, min_prefix=64, hibernate_holders=True, hibernate_idle_seconds=10.0,
                            spill=PrefixSpillConfig(enabled=True, path=str(d), max_mib=2, idle_seconds=100.0))
    pc = PrefixCache(eng, cfg)
    assert pc.spill_dir == str(d) and not (d / "ls-spill-999-1-1.kvspill").exists() and (d / "keep.txt").exists()
    prompts = [[100 * k + i % 50 for i in range(64)] for k in range(3)]
    holders = []
    for p in prompts:
        sid = eng.create_sequence()
        eng.prefill(sid, p)
        holders.append(pc.register(sid, p))
        eng.free_sequence(sid)
    t0 = __import__("time").monotonic()
    assert pc.idle_sweep(t0 + 1) == {"hibernated": 0, "spilled": 0}                    # nobody idle long enough
    assert pc.idle_sweep(t0 + 20) == {"hibernated": 3, "spilled": 0} and set(eng.hibernated) == set(holders)
    # second hop: one per sweep, LRU first; 4 pages of 300 KiB = 1.2 MB each under a 2 MiB cap -> the third spill drops the first
    assert pc.idle_sweep(t0 + 200)["spilled"] == 1 and list(eng.spilled) == [holders[0]]
    pc.idle_sweep(t0 + 201)
    pc.idle_sweep(t0 + 202)
    assert pc.spill_stats["cap_evictions"] >= 1 and holders[0] not in eng.seqs            # dropped with its file
    assert sum(b for _, b in pc._spilled.values()) <= 2 << 20
    assert len([f for f in os.listdir(d) if f.endswith(".kvspill")]) == len(pc._spilled)
    # a hit on a spilled holder brings it back through the engine
    spilled = next(iter(pc._spilled))
    k = holders.index(spilled)
    sid, n = pc.fork_from(prompts[k] + [7])
    assert sid is not None and n == 64 and spilled not in pc._spilled and spilled not in eng.spilled
    eng.free_sequence(sid)
    # a lost file is a cache miss: the holder is dropped, the request will prefill
    for h in list(eng.hibernated):
        pc._hit_time[h] = t0
    pc.idle_sweep(t0 + 500)
    victim = next(iter(pc._spilled))
    os.remove(pc._spilled[victim][0])
    k = holders.index(victim)
    misses = pc.misses
    assert pc.fork_from(prompts[k] + [7]) == (None, 0)
    assert pc.misses == misses + 1 and victim not in eng.seqs and pc.spill_stats["lost_files"] == 1
    # an unwritable directory disables the second hop, the first still works
    pc2 = PrefixCache(Tiered(max_seqs=4, max_ctx=256, page=16),
                      PrefixCacheConfig(hibernate_holders=True, spill=PrefixSpillConfig(enabled=True, path="/proc/definitely/not/writable")))
    assert pc2.spill_dir is None


def test_a_sticky_device_error_is_recorded_once_and_stops_admission():
    """Host-side injection: the engine's step raises what a lost CUDA context raises.  The failing request and everything queued
    behind it end with the cause, /health turns 503, new requests are refused at once; an ordinary request error or a bounded
    device wait that ran out does not trip it."""
    from fastapi.testclient import TestClient
    from layerstorm_b200.runtime.null_engine import NullEngine
    from layerstorm_b200.serving.http_server import LayerStormServer, ServerConfig
    from layerstorm_b200.serving.orchestrator import InferenceRequest, Orchestrator, SamplingParams, is_gpu_fatal
    from layerstorm_b200.serving.tokenizer import TokenizerWrapper

    class DeviceWaitError(RuntimeError):
        pass

    assert is_gpu_fatal(RuntimeError("CUDA error: an illegal memory access was encountered"))
    assert is_gpu_fatal(RuntimeError("CUDA error: unspecified launch failure"))
    assert not is_gpu_fatal(ValueError("prompt too long")) and not is_gpu_fatal(DeviceWaitError("all-reduce wait ran out (code 21)"))

    class Flaky(NullEngine):
        mode = None

        def decode(self, sids, tokens, **kw):
            if self.mode == "request":
                self.mode = None
                raise ValueError("bad request state")
            if self.mode == "fatal":
                raise RuntimeError("CUDA error: an illegal memory access was encountered")
            return super().decode(sids, tokens, **kw)

    eng = Flaky(vocab=300)
    orch = Orchestrator(eng, eos_token_ids=[1])

    import itertools
    ids = itertools.count()

    def req(n=4):
        return InferenceRequest(f"r{next(ids)}", [5, 6, 7, 8], SamplingParams(max_tokens=n, ignore_eos=True))

    eng.mode = "request"
    r0 = req()
    orch.submit_request(r0)
    orch.step()
    assert r0.error and orch.gpu_fatal is None                                   # an ordinary failure: the next request is served
    r1 = req()
    orch.submit_request(r1)
    orch.step()
    assert r1.error is None and len(r1.output_ids) == 4
    eng.mode = "fatal"
    r2, r3 = req(), req()
    orch.submit_request(r2)
    orch.submit_request(r3)
    orch.step()
    assert "illegal memory access" in r2.error and orch.gpu_fatal and r3.done.is_set() and r3.error.startswith("gpu_fatal")
    assert orch.queued() == 0
    r4 = req()
    orch.submit_request(r4)                                                       # refused at once, never queued
    assert r4.done.is_set() and r4.error.startswith("gpu_fatal") and orch.queued() == 0
    server = LayerStormServer(orch, TokenizerWrapper(None, vocab_limit=300), ServerConfig(model_name="t"))
    c = TestClient(server.app)
    h = c.get("/health")
    assert h.status_code == 503 and "gpu_fatal" in h.text
    assert c.post("/v1/completions", json={"prompt": "hi", "max_tokens": 2}).status_code == 503


def test_continuous_batching_gives_each_request_its_sequential_tokens():
    """Plain greedy requests decode together (one engine step per token of all of them), join after their own prefill and leave
    when they finish; every request gets exactly the tokens it gets when served alone; a request that needs its own decode arm
    (log-probabilities) is served alone in arrival order; a cancelled request leaves the batch."""
    import itertools
    from layerstorm_b200.runtime.null_engine import NullEngine
    from layerstorm_b200.serving.orchestrator import InferenceRequest, Orchestrator, SamplingParams
    ids = itertools.count()

    def make(n_prompt, n_gen, **kw):
        prompt = [(13 * next(ids) + 7 * i) % 250 + 4 for i in range(n_prompt)]
        return InferenceRequest(f"r{next(ids)}", prompt, SamplingParams(max_tokens=n_gen, ignore_eos=True, **kw))

    specs = [(20, 9), (70, 3), (33, 14), (5, 1), (90, 6), (40, 11)]
    reqs = [make(a, b) for a, b in specs]
    seq = Orchestrator(NullEngine(vocab=300, max_seqs=16), eos_token_ids=[1])
    want = []
    for r in reqs:
        c = InferenceRequest(r.request_id + "s", list(r.prompt_ids), r.params)
        seq.submit_request(c)
        seq.step()
        want.append(list(c.output_ids))
    eng = NullEngine(vocab=300, max_seqs=16)
    orch = Orchestrator(eng, eos_token_ids=[1], max_batch=4)
    for r in reqs[:5]:
        orch.submit_request(r)
    lp = make(12, 4, logprobs=2)                        # not batchable: waits for the batch to drain, then runs alone
    orch.submit_request(lp)
    orch.submit_request(reqs[5])
    peak = 0
    for _ in range(400):
        if not orch.step():
            break
        peak = max(peak, len(orch.running))
    assert all(r.done.is_set() and r.error is None for r in reqs + [lp])
    assert [list(r.output_ids) for r in reqs] == want
    assert len(lp.output_ids) == 4 and peak >= 3 and orch.served == 7 and not orch.running and len(eng.seqs) == orch.prefix.holders()
    assert orch.batched_steps < sum(b for _, b in specs) - len(specs)            # tokens were produced together, not one request at a time
    # the request behind the unbatchable one started only after it: arrival order is kept
    assert lp.stats.t_done <= reqs[5].stats.t_first_token
    # cancellation of a running request frees its sequence at its next token; the others go on
    a, b = make(10, 50), make(10, 8)
    orch.submit_request(a)
    orch.submit_request(b)
    for _ in range(4):
        orch.step()
    assert orch.cancel_request(a.request_id)
    for _ in range(40):
        if not orch.step():
            break
    assert a.done.is_set() and a.finish_reason == "cancelled" and len(a.output_ids) < 50 and len(b.output_ids) == 8 and len(eng.seqs) == orch.prefix.holders()


def test_a_joining_requests_prompt_is_prefilled_in_slices_between_decode_steps():
    """Continuous batching with a long prompt arriving while another request decodes: the prompt goes in slices, the running
    request gets a token between every two slices (it never waits for the whole prompt), and both end with their sequential tokens."""
    from layerstorm_b200.runtime.null_engine import NullEngine
    from layerstorm_b200.serving.orchestrator import InferenceRequest, Orchestrator, SamplingParams
    events = []
    short = InferenceRequest("short", [9, 8, 7, 6, 5], SamplingParams(max_tokens=40, ignore_eos=True), on_token=lambda t, i: events.append("s"))
    long_prompt = [(11 * i) % 240 + 4 for i in range(200)]
    long = InferenceRequest("long", long_prompt, SamplingParams(max_tokens=5, ignore_eos=True), on_token=lambda t, i: events.append("L"))
    seq = Orchestrator(NullEngine(vocab=300), eos_token_ids=[1])
    want = {}
    for r in (short, long):
        c = InferenceRequest(r.request_id, list(r.prompt_ids), r.params)
        seq.submit_request(c)
        seq.step()
        want[r.request_id] = list(c.output_ids)

    class Counting(NullEngine):
        def prefill(self, sid, tokens, want_logits=False):
            events.append(f"p{len(tokens)}")
            return super().prefill(sid, tokens, want_logits)

    orch = Orchestrator(Counting(vocab=300), eos_token_ids=[1], max_batch=4, prefill_slice_tokens=32)
    orch.submit_request(short)
    orch.step()
    orch.step()
    orch.submit_request(long)
    for _ in range(200):
        if not orch.step():
            break
    assert list(short.output_ids) == want["short"] and list(long.output_ids) == want["long"]
    slices = [e for e in events if e.startswith("p")]
    assert slices == ["p5"] + ["p32"] * 6 + ["p8"] and orch.prefill_slices == 8        # 200 = 6 x 32 + 8
    # between two consecutive slices of the long prompt the short request produced exactly one token
    idx = [i for i, e in enumerate(events) if e.startswith("p")][1:]
    assert all(events[a + 1: b] == ["s"] for a, b in zip(idx, idx[1:]))
    assert events.index("L") > idx[-1]


def test_the_serving_loop_sweeps_idle_prefix_holders_between_requests(tmp_path):
    """The orchestrator's own loop (a thread, as in the server) runs the prefix cache's idle sweep when it has nothing to serve:
    holders of finished requests hibernate and spill without any request asking for it, and a later request with the same prefix
    still hits the cache."""
    import threading
    import time as _time
    import torch
    from layerstorm_b200.runtime.null_engine import NullEngine
    from layerstorm_b200.serving.orchestrator import InferenceRequest, Orchestrator, SamplingParams
    from layerstorm_b200.serving.prefix_cache import PrefixCacheConfig, PrefixSpillConfig

    class Tiered(NullEngine):
        def __init__(self, **kw):
            super().__init__(**kw)
            self.hibernated, self.spilled = {}, {}
            self.cold_kv, self.cold_idx = {0: torch.zeros(1, 16, 64, dtype=torch.uint8)}, {}

        def hibernate(self, sid):
            self.hibernated[sid] = [0] * ((self.seqs[sid].length + self.page - 1) // self.page)
            return len(self.hibernated[sid])

        def spill(self, sid, path):
            n = len(self.hibernated.pop(sid)) * 1024
            open(path, "wb").write(b"x")
            self.spilled[sid] = (path, n)
            return n

        def fork_sequence(self, parent, prefix_len=None):
            self.spilled.pop(parent, None)
            self.hibernated.pop(parent, None)
            return super().fork_sequence(parent, prefix_len)

    eng = Tiered(vocab=300, max_seqs=8)
    pcc = PrefixCacheConfig(grid=64, min_prefix=64, hibernate_holders=True, hibernate_idle_seconds=0.0,
                            spill=PrefixSpillConfig(enabled=True, path=str(tmp_path), max_mib=1, idle_seconds=0.0))
    orch = Orchestrator(eng, eos_token_ids=[1], prefix_cache=pcc)
    t = threading.Thread(target=orch.run, daemon=True)
    t.start()
    try:
        prompt = [(7 * i) % 250 + 4 for i in range(80)]
        r1 = InferenceRequest("a", list(prompt), SamplingParams(max_tokens=3, ignore_eos=True))
        orch.submit_request(r1)
        assert r1.done.wait(5)
        deadline = _time.time() + 8
        while _time.time() < deadline and not eng.spilled:          # two idle sweeps, one second apart: hibernate, then spill
            _time.sleep(0.1)
        assert eng.spilled and orch.prefix.spill_stats["spilled"] == 1 and not getattr(orch, "last_sweep_error", None)
        r2 = InferenceRequest("b", list(prompt) + [9, 9], SamplingParams(max_tokens=3, ignore_eos=True))
        orch.submit_request(r2)
        assert r2.done.wait(5) and r2.error is None and r2.stats.cached_tokens == 64
    finally:
        orch.shutdown()
        t.join(timeout=5)


def test_a_degraded_prefill_is_never_cached_and_is_retried_within_its_budget():
    """An engine that reports a degraded step during a prefill (an expert missed its fetch deadline): the orchestrator does not
    register a prefix holder for those KV rows, runs the request again while it has retry budget - nothing was emitted yet - and
    counts what it did; without budget the degraded answer is delivered and marked."""
    from layerstorm_b200.runtime.null_engine import NullEngine
    from layerstorm_b200.serving.orchestrator import InferenceRequest, Orchestrator, SamplingParams

    class Flaky(NullEngine):
        degraded_steps = 0
        bad_prefills = 0

        def prefill(self, sid, tokens, want_logits=False):
            if self.bad_prefills > 0:
                self.bad_prefills -= 1
                self.degraded_steps += 1
            return super().prefill(sid, tokens, want_logits)

    prompt = [(5 * i) % 200 + 4 for i in range(70)]

    def request(name):
        seen = []
        return InferenceRequest(name, list(prompt), SamplingParams(max_tokens=4, ignore_eos=True), on_token=lambda t, i: seen.append(t)), seen

    eng = Flaky(vocab=300)
    orch = Orchestrator(eng, eos_token_ids=[1], degraded_retry_max=1)
    eng.bad_prefills = 1
    r, seen = request("a")
    orch.submit_request(r)
    orch.step()
    assert r.error is None and r.stats.degraded_retries == 1 and r.stats.moe_degraded_steps == 0 and len(seen) == 4      # emitted once, from the clean attempt
    assert orch.degraded_retries_total == 1 and orch.degraded_delivered_total == 0 and orch.prefix.holders() == 1
    # two degraded prefills in a row with a budget of one: the second attempt is delivered, marked, and not cached
    orch.prefix.clear()
    eng.bad_prefills = 2
    r2, seen2 = request("b")
    orch.submit_request(r2)
    orch.step()
    assert r2.error is None and r2.stats.degraded_retries == 1 and r2.stats.moe_degraded_steps == 1 and len(seen2) == 4
    assert orch.degraded_delivered_total == 1 and orch.prefix.holders() == 0
    assert len(eng.seqs) == 0                                  # abandoned attempts freed their sequences
    # retries off (the default): delivered first try, marked
    o2 = Orchestrator(Flaky(vocab=300), eos_token_ids=[1])
    o2.engine.bad_prefills = 1
    r3, _ = request("c")
    o2.submit_request(r3)
    o2.step()
    assert r3.stats.degraded_retries == 0 and r3.stats.moe_degraded_steps == 1 and o2.prefix.holders() == 0


def test_a_request_that_finds_no_kv_pages_waits_for_a_running_one_to_finish():
    """Continuous batching under memory pressure: a joining request that cannot get KV pages (or a sequence slot) while others are
    decoding goes back to the head of the queue and is admitted when one of them has finished; alone on the engine the same
    shortage is an error."""
    from layerstorm_b200.runtime.null_engine import NullEngine
    from layerstorm_b200.serving.orchestrator import InferenceRequest, Orchestrator, SamplingParams
    from layerstorm_b200.serving.prefix_cache import PrefixCacheConfig
    eng = NullEngine(vocab=300, max_seqs=8, page=16, num_pages=10)       # 160 tokens of KV in total
    orch = Orchestrator(eng, eos_token_ids=[1], max_batch=4, prefix_cache=PrefixCacheConfig(enabled=False))
    a = InferenceRequest("a", [7] * 60, SamplingParams(max_tokens=20, ignore_eos=True))     # 5 pages
    b = InferenceRequest("b", [8] * 60, SamplingParams(max_tokens=30, ignore_eos=True))     # 5 pages (6 after 20 tokens)
    c = InferenceRequest("c", [9] * 40, SamplingParams(max_tokens=5, ignore_eos=True))      # 3 pages: does not fit beside a and b
    for r in (a, b, c):
        orch.submit_request(r)
    for _ in range(300):
        if not orch.step():
            break
    assert all(r.done.is_set() for r in (a, b, c)) and a.error is None and c.error is None and len(c.output_ids) == 5
    assert orch.admission_waits >= 1 and c.stats.t_first_token >= a.stats.t_done - 1e-3     # c got in only after a had finished
    assert b.error is None and len(b.output_ids) == 30
    # alone on the engine a prompt that cannot fit is an error, not an endless wait
    big = InferenceRequest("big", [5] * 400, SamplingParams(max_tokens=2, ignore_eos=True))
    orch.submit_request(big)
    for _ in range(20):
        if not orch.step():
            break
    assert big.done.is_set() and big.error is not None


def test_decode_that_runs_out_of_kv_pages_preempts_the_youngest_request_and_resumes_it():
    """Two requests whose prompts fit but whose generations outgrow the pool: the younger one gives its pages back in mid-decode, joins
    again behind what it has produced, and both deliver exactly the tokens they deliver when served alone."""
    from layerstorm_b200.runtime.null_engine import NullEngine
    from layerstorm_b200.serving.orchestrator import InferenceRequest, Orchestrator, SamplingParams
    from layerstorm_b200.serving.prefix_cache import PrefixCacheConfig

    def serve(reqs, pages, batch):
        eng = NullEngine(vocab=300, max_seqs=8, page=16, num_pages=pages)
        orch = Orchestrator(eng, eos_token_ids=[1], max_batch=batch, prefix_cache=PrefixCacheConfig(enabled=False))
        for r in reqs:
            orch.submit_request(r)
        for _ in range(1000):
            if not orch.step():
                break
        return orch

    def mk():
        return [InferenceRequest("a", [7] * 30, SamplingParams(max_tokens=60, ignore_eos=True)),      # 2 pages -> 6 pages
                InferenceRequest("b", [8, 9] * 15, SamplingParams(max_tokens=60, ignore_eos=True))]
    alone = mk()
    serve(alone, 64, 1)
    tight = mk()
    orch = serve(tight, 9, 4)                                                                        # 12 pages would be needed side by side
    assert orch.preemptions >= 1 and tight[1].stats.preemptions >= 1 and tight[0].stats.preemptions == 0
    for x, y in zip(alone, tight):
        assert y.error is None and y.output_ids == x.output_ids and len(y.output_ids) == 60
    assert orch.engine.free_page_count() == 9


def test_health_reports_the_draft_side():
    from fastapi.testclient import TestClient
    from layerstorm_b200.serving.http_server import LayerStormServer, ServerConfig
    from layerstorm_b200.speculation.combiner import DepthPolicy, DraftCombiner, DraftSource, UtilityScorer
    from layerstorm_b200.speculation.prompt_lookup import IncrementalPromptLookup

    class Wrong:
        def propose(self, ctx, g): return [3] * g
    tok = TokenizerWrapper()
    eng = NullEngine(vocab=tok.vocab_size)
    comb = DraftCombiner([DraftSource("prompt_lookup", IncrementalPromptLookup(), cost=0.0), DraftSource("model", Wrong(), cost=0.1)])
    orch = Orchestrator(eng, eos_token_ids=tok.eos_token_ids, tokenizer=tok, draft=comb, speculation_depth=3,
                        depth_policy=DepthPolicy(UtilityScorer("ema", max_depth=3), None, max_depth=3, alpha=0.5))
    srv = LayerStormServer(orch, tok, ServerConfig(model_name="m"))
    c = TestClient(srv.app)
    s0 = c.get("/health").json()["speculation"]
    assert s0["depth"] == 3 and s0["sources"] == {"prompt_lookup": 0.5, "model": 0.5} and s0["last_source"] is None and s0["acceptance"] == 0.6
    r = InferenceRequest("h", list(range(5, 30)), SamplingParams(max_tokens=20, ignore_eos=True))
    orch.submit_request(r)
    assert orch.step() and r.error is None
    s1 = c.get("/health").json()["speculation"]
    assert s1["last_source"] == "model" and s1["sources"]["model"] < 0.5 and s1["acceptance"] < 0.3 and s1["plain_rounds"] > 0
    # no draft: nothing to report
    plain = LayerStormServer(Orchestrator(NullEngine(vocab=tok.vocab_size), eos_token_ids=tok.eos_token_ids, tokenizer=tok), tok, ServerConfig(model_name="m"))
    assert TestClient(plain.app).get("/health").json()["speculation"] == {}
