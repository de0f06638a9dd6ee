"""Serving stack on the GPU engine: HTTP completions through the CLI-built server, lossless speculative decoding with a
model draft on its own engine, prefix-cache reuse."""
import threading

import pytest
import torch

pytestmark = pytest.mark.gpu


def _engine(name="tiny-mla-moe", seed=0, **kw):
    from layerstorm_b200.models.config import get_preset
    from layerstorm_b200.models.device_model import DeviceModel
    from layerstorm_b200.models.weights import init_weights
    from layerstorm_b200.runtime.engine import Engine
    cfg = get_preset(name)
    m = DeviceModel.from_state_dict(cfg, init_weights(cfg, seed), "cuda", kv_fmt="bf16", page=16)
    return cfg, Engine(m, max_seqs=6, max_ctx=256, prefill_chunk=32, max_batch=1, **kw)


def test_http_completions_on_the_gpu_engine():
    from fastapi.testclient import TestClient
    from layerstorm_b200.cli import serve
    args = serve.build_parser().parse_args(["--model", "tiny-mla-moe", "--random-weights", "--tokenizer-mode", "byte", "--model-name", "tiny",
                                            "--max-concurrent", "2", "--max-sequence-length", "256"])
    cfg, shape, ckpt, _ = serve.resolve_config(args)
    cfg["memory"]["kv_cache"]["page_size_tokens"] = 16
    eng = serve.build_engine(cfg, shape, ckpt, args)
    server, orch = serve.build_server(cfg, shape, ckpt, eng, args)
    t = threading.Thread(target=orch.run, daemon=True)
    t.start()
    try:
        c = TestClient(server.app)
        assert c.get("/v1/models").json()["data"][0]["id"] == "tiny"
        body = {"prompt": "hello world, hello world", "max_tokens": 8, "temperature": 0, "ignore_eos": True}
        r1 = c.post("/v1/completions", json=body).json()
        r2 = c.post("/v1/completions", json=body).json()
        assert r1["usage"]["completion_tokens"] == 8 and r1["choices"][0]["text"] == r2["choices"][0]["text"]      # greedy is reproducible
        r3 = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "hi"}], "max_tokens": 4, "ignore_eos": True})
        assert r3.status_code == 200 and r3.json()["choices"][0]["message"]["role"] == "assistant"
        lines = []
        with c.stream("POST", "/v1/completions", json=dict(body, stream=True)) as s:
            for ln in s.iter_lines():
                if ln.startswith("data: "):
                    lines.append(ln)
        assert lines[-1] == "data: [DONE]" and len(lines) >= 3
    finally:
        orch.shutdown()
        t.join(timeout=5)


def test_speculative_decoding_with_model_draft_is_lossless():
    from layerstorm_b200.serving.orchestrator import InferenceRequest, Orchestrator, SamplingParams
    from layerstorm_b200.speculation import DraftCombiner, DraftSource, EngineDraft, PromptLookupDraft
    cfg, target = _engine(seed=3, use_graph=False)
    _, draft_eng = _engine(seed=3, use_graph=True)              # same weights => the draft is always right
    _, other_eng = _engine(seed=4, use_graph=True)              # different weights => mostly wrong drafts
    prompt = torch.randint(0, cfg.vocab, (24,), generator=torch.Generator().manual_seed(1)).tolist()
    ref = InferenceRequest("ref", list(prompt), SamplingParams(max_tokens=20, ignore_eos=True))
    o = Orchestrator(target)
    o.submit_request(ref); o.step()
    for name, de in (("same", draft_eng), ("other", other_eng)):
        comb = DraftCombiner([DraftSource("prompt_lookup", PromptLookupDraft(2, 4, 4), cost=0.0), DraftSource("model", EngineDraft(de, 4), cost=0.1)])
        req = InferenceRequest(name, list(prompt), SamplingParams(max_tokens=20, ignore_eos=True))
        s = Orchestrator(target, draft=comb, speculation_depth=4)
        s.submit_request(req); s.step()
        assert req.output_ids == ref.output_ids, name            # lossless whatever the draft proposes
        assert req.stats.spec_rounds > 0
        if name == "same":
            assert req.stats.spec_accepted >= 3 * req.stats.spec_rounds - 4


def test_prefix_cache_hit_on_the_gpu_engine():
    from layerstorm_b200.serving.orchestrator import InferenceRequest, Orchestrator, SamplingParams
    from layerstorm_b200.serving.prefix_cache import PrefixCacheConfig
    cfg, eng = _engine(seed=5, use_graph=False)
    orch = Orchestrator(eng, prefix_cache=PrefixCacheConfig(enabled=True, grid=16, min_prefix=16))
    base = torch.randint(0, cfg.vocab, (64,), generator=torch.Generator().manual_seed(2)).tolist()
    outs = []
    for i, tail in enumerate(([7, 8, 9], [7, 8, 9], [10, 11])):
        req = InferenceRequest(f"r{i}", base + tail, SamplingParams(max_tokens=6, ignore_eos=True))
        orch.submit_request(req); orch.step()
        outs.append((req.output_ids, req.stats.cached_tokens))
    assert outs[0][0] == outs[1][0] and outs[0][1] == 0 and outs[1][1] >= 64 and outs[2][1] >= 64
    cold = Orchestrator(_engine(seed=5, use_graph=False)[1], prefix_cache=PrefixCacheConfig(enabled=False))
    req = InferenceRequest("cold", base + [10, 11], SamplingParams(max_tokens=6, ignore_eos=True))
    cold.submit_request(req); cold.step()
    assert req.output_ids == outs[2][0]                          # cache on == cache off


def test_speculation_on_a_recurrent_state_model_is_lossless_and_decided_on_the_device():
    """glm5_next (KDA layers): a speculative round is verified on the device (arg-max per row + prefix count, 8 bytes back) and a
    partly rejected round is undone through the recurrent-state anchor + replay.  Tokens equal plain greedy decoding whatever
    the draft proposes; with a perfect draft every round accepts all drafted tokens."""
    from layerstorm_b200.serving.orchestrator import InferenceRequest, Orchestrator, SamplingParams
    from layerstorm_b200.speculation import EngineDraft
    cfg, target = _engine("tiny-glm5-next", seed=3, use_graph=False)
    assert target.has_recurrent_state
    _, same = _engine("tiny-glm5-next", seed=3, use_graph=False)
    _, other = _engine("tiny-glm5-next", seed=4, use_graph=False)
    prompt = torch.randint(0, cfg.vocab, (40,), generator=torch.Generator().manual_seed(1)).tolist()
    ref = InferenceRequest("ref", list(prompt), SamplingParams(max_tokens=24, ignore_eos=True))
    o = Orchestrator(target)
    o.submit_request(ref); o.step()
    for name, de in (("same", same), ("other", other)):
        d2h0 = target.d2h_bytes
        req = InferenceRequest(name, list(prompt), SamplingParams(max_tokens=24, ignore_eos=True))
        s = Orchestrator(target, draft=EngineDraft(de, 4), speculation_depth=4)
        s.submit_request(req); s.step()
        assert req.error is None, req.error
        assert req.output_ids == ref.output_ids, name
        assert req.stats.spec_rounds > 0
        assert target.d2h_bytes - d2h0 < 64 * (req.stats.spec_rounds + 30), "verify rounds must not copy logits to the host"
        if name == "same":
            assert req.stats.spec_accepted >= 3 * req.stats.spec_rounds - 4
        else:
            assert req.stats.spec_accepted < 4 * req.stats.spec_rounds           # some round was rolled back through the anchor


def test_sampled_requests_draw_on_the_device_and_repeat_for_a_fixed_seed():
    from layerstorm_b200.serving.orchestrator import InferenceRequest, Orchestrator, SamplingParams
    cfg, eng = _engine("tiny-glm5-next", seed=6, use_graph=True)
    orch = Orchestrator(eng)
    prompt = torch.randint(0, cfg.vocab, (20,), generator=torch.Generator().manual_seed(4)).tolist()
    outs = []
    for seed in (11, 11, 12):
        d2h0 = eng.d2h_bytes
        req = InferenceRequest(f"s{seed}", list(prompt), SamplingParams(max_tokens=16, ignore_eos=True, temperature=1.0, top_k=40, top_p=0.95, seed=seed))
        orch.submit_request(req); orch.step()
        assert req.error is None, req.error
        assert eng.d2h_bytes - d2h0 < 16 * 64, "sampled decode must not copy the vocabulary's logits to the host"
        outs.append(req.output_ids)
    assert outs[0] == outs[1] and outs[0] != outs[2] and len(outs[0]) == 16
    greedy = InferenceRequest("g", list(prompt), SamplingParams(max_tokens=16, ignore_eos=True))
    orch.submit_request(greedy); orch.step()
    assert greedy.output_ids != outs[0]


def test_decode_reports_the_steps_confidence_from_the_device():
    """``Engine.decode(confidence=True)``: top-1 probability and entropy of the step's distribution come back with the token (8 bytes per row)
    and equal the softmax of the logits; a confidence-gated draft stops at the first token below its threshold."""
    import torch
    from layerstorm_b200.models.config import get_preset
    from layerstorm_b200.models.device_model import DeviceModel
    from layerstorm_b200.models.weights import init_weights
    from layerstorm_b200.runtime.engine import Engine
    from layerstorm_b200.speculation.model_draft import EngineDraft
    cfg = get_preset("tiny-mla-moe")
    m = DeviceModel.from_state_dict(cfg, init_weights(cfg, 5), "cuda", kv_fmt="bf16", page=16)
    eng = Engine(m, max_seqs=2, max_ctx=128, prefill_chunk=16, max_batch=1, use_graph=True)
    assert eng.supports_confidence
    sid = eng.create_sequence()
    prompt = torch.randint(0, cfg.vocab, (20,), generator=torch.Generator().manual_seed(1)).tolist()
    tok = eng.prefill(sid, prompt)
    toks, conf = eng.decode([sid], [tok], confidence=True)
    lg = eng.ws_decode[1].logits[0].float()
    p = torch.softmax(lg, 0)
    assert abs(conf[0][0] - float(p.max())) < 1e-4
    import math
    ent = float(-(p * torch.log(p.clamp_min(1e-30))).sum()) / math.log(cfg.vocab)          # the kernel reports entropy / ln(vocabulary)
    assert abs(conf[0][1] - ent) < 1e-3
    assert toks[0] == int(lg.argmax())
    # gated drafting: an impossible threshold stops at once, a zero threshold drafts the full depth
    ctx = prompt + [tok]
    d_all = EngineDraft(Engine(m, max_seqs=2, max_ctx=128, prefill_chunk=16, max_batch=1), max_gamma=4, min_confidence=0.0)
    d_none = EngineDraft(Engine(m, max_seqs=2, max_ctx=128, prefill_chunk=16, max_batch=1), max_gamma=4, min_confidence=1.1)
    assert len(d_all.propose(ctx, 4)) == 4
    assert d_none.propose(ctx, 4) == [] and d_none.early_stops == 1


@pytest.mark.parametrize("name", ["tiny-mla-moe", "tiny-glm5-next"])
def test_self_speculative_draft_with_layer_skipping_is_lossless_on_the_gpu(name):
    """The target drafts for itself with fewer experts AND with layers left out; the skip set comes from the cosine similarities the draft
    steps record on the device.  Verification by the full model keeps the output identical to plain greedy decoding."""
    from layerstorm_b200.models.config import get_preset
    from layerstorm_b200.models.device_model import DeviceModel
    from layerstorm_b200.models.weights import init_weights
    from layerstorm_b200.runtime.engine import Engine
    from layerstorm_b200.serving.orchestrator import InferenceRequest, Orchestrator, SamplingParams
    from layerstorm_b200.speculation.self_draft import SelfSpeculativeDraft
    cfg = get_preset(name)
    m = DeviceModel.from_state_dict(cfg, init_weights(cfg, 3), "cuda", kv_fmt="bf16", page=16)
    prompt = list(range(7, 31))

    def run(draft_for=None):
        eng = Engine(m, max_seqs=2, max_ctx=128, prefill_chunk=16, max_batch=1)
        draft = draft_for(eng) if draft_for else None
        orch = Orchestrator(eng, draft=draft, speculation_depth=3) if draft else Orchestrator(eng)
        req = InferenceRequest("r", prompt, SamplingParams(max_tokens=14, ignore_eos=True))
        orch.submit_request(req)
        assert orch.step() and req.error is None
        return req, draft

    plain, _ = run()
    # a threshold below any cosine: every unprotected layer the policy may skip is skipped from the second round on
    skip_cfg = {"enabled": True, "threshold": -1.0, "min_acceptance_rate_to_enable": 0.0, "no_skip_first": 1, "no_skip_last": 1,
                "target_skip_fraction": 0.5}
    spec, draft = run(lambda eng: SelfSpeculativeDraft(eng, {"draft_expert_count": 2, "adaptive_exit_enabled": False}, max_gamma=3, layer_skip=skip_cfg))
    assert spec.output_ids == plain.output_ids
    assert spec.stats.spec_rounds > 0 and draft.failures == 0
    assert draft.skip_set and draft.skipped_layer_steps > 0                 # layers were really left out of draft steps
    assert all(0 < l < cfg.n_layers - 1 for l in draft.skip_set)
    sims = draft.engine.layer_similarities()
    assert sims and all(-1.001 <= v <= 1.001 for v in sims.values())


def test_cosine_similarity_kernel():
    from layerstorm_b200.ops import _native as nat
    g = torch.Generator(device="cuda").manual_seed(2)
    a = torch.randn(5, 1000, device="cuda", generator=g).to(torch.bfloat16)
    b = (a.float() * 0.7 + torch.randn(5, 1000, device="cuda", generator=g) * 0.5).to(torch.bfloat16)
    b[3] = 0
    out = torch.full((5,), 9.0, device="cuda")
    nat.call("lsb_cosine_sim", a, b, 5, 1000, 1000, 1000, out)
    torch.cuda.synchronize()
    ref = torch.nn.functional.cosine_similarity(a.float(), b.float(), dim=1)
    assert float(out[3]) == 0.0
    keep = torch.tensor([0, 1, 2, 4], device="cuda")
    assert torch.allclose(out[keep], ref[keep], atol=1e-5)


@pytest.mark.parametrize("name", ["tiny-mla-moe", "tiny-deepseek-v32"])
def test_device_mtp_block_matches_the_reference_and_stays_in_step_through_speculation(name):
    """The multi-token-prediction block on the device: after a chunked prefill and after every speculative round (accepted or
    rejected drafts, plain decode steps in between) its proposal equals the fp32 reference's, which recomputes the main stream and
    the block from scratch; greedy speculation with it reproduces plain greedy decoding token for token."""
    import dataclasses
    from layerstorm_b200.models.config import get_preset
    from layerstorm_b200.models.device_model import DeviceModel
    from layerstorm_b200.models.mtp import mtp_block
    from layerstorm_b200.models.reference import Oracle
    from layerstorm_b200.models.weights import init_weights
    from layerstorm_b200.runtime.engine import Engine
    cfg = dataclasses.replace(get_preset(name), n_mtp=1)
    w = init_weights(cfg, 3)
    m = DeviceModel.from_state_dict(cfg, w, "cuda", kv_fmt="bf16", page=16, expert_quant="bf16", dense_quant="bf16", with_mtp=True)
    assert len(m.mtp_layers) == 1
    oracle = Oracle(cfg, m.effective_state_dict())
    g = torch.Generator().manual_seed(4)
    T = 27                                             # below index_topk: dense selection in the main model on both sides
    prompt = torch.randint(0, cfg.vocab, (T,), generator=g).tolist()

    def ref_draft(context):
        """logits of the block at the last fed position: main stream over context[:-1], token ahead = context[1:]."""
        n = len(context) - 1
        _, hidden = oracle.forward(torch.tensor(context[:n]), return_hidden=True)
        logits, _ = mtp_block(oracle, 0, hidden, context[1: n + 1])
        return logits[-1]

    plain = Engine(m, max_seqs=2, max_ctx=128, prefill_chunk=8, max_batch=1, use_graph=False)
    sid0 = plain.create_sequence()
    tok = plain.prefill(sid0, prompt)
    want = [tok]
    for _ in range(9):
        want.append(plain.decode([sid0], [want[-1]])[0])
    plain.free_sequence(sid0)

    eng = Engine(m, max_seqs=3, max_ctx=128, prefill_chunk=8, max_batch=1, use_graph=False)
    eng.enable_mtp()
    sid = eng.create_sequence()
    tok = eng.prefill(sid, prompt)
    assert tok == want[0]
    got, ctx = [tok], prompt + [tok]
    rounds = accepted = 0
    while len(got) < 10:
        d = eng.mtp_draft(sid, tok)
        assert len(d) == 1
        ref = ref_draft(ctx)
        lg = eng.mtp.last_ws.logits[0].float().cpu()
        assert float((lg - ref).abs().max() / (ref.abs().max() + 1e-9)) < 3e-2
        assert d[0] == int(ref.argmax())
        if rounds % 3 == 2:
            tok = eng.decode([sid], [tok])[0]          # a plain step in between: the block catches up on its own
            new = [tok]
        else:
            n_acc, nxt = eng.verify_greedy(sid, tok, d)
            accepted += n_acc
            new = d[:n_acc] + [nxt]
            tok = nxt
        rounds += 1
        got += new
        ctx += new
    assert got[:10] == want[:10]
    assert eng.mtp.block_rows >= T - 1 + rounds
    # a fork at the frontier keeps the block in step; a fork below it proposes nothing (and never a wrong cache)
    child = eng.fork_sequence(sid)
    assert eng.mtp_draft(child, tok) == eng.mtp_draft(sid, tok)
    low = eng.fork_sequence(sid, (eng.seq_len(sid) // 2))
    assert eng.mtp_draft(low, tok) == []


def test_serve_streams_experts_when_the_configuration_keeps_part_of_them_in_hbm():
    """``autoconfig.vram_expert_ratio`` < 1 in the configuration: the server's own boot path builds the expert streamer (layer by
    layer), the engine runs eager steps through it and a request gives the tokens of the fully resident server."""
    from layerstorm_b200.cli import serve
    from layerstorm_b200.serving.orchestrator import InferenceRequest, SamplingParams

    def boot(ratio):
        args = serve.build_parser().parse_args(["--model", "tiny-mla-moe", "--random-weights", "--tokenizer-mode", "byte", "--max-concurrent", "2",
                                                "--max-sequence-length", "256"])
        cfg, shape, ckpt, _ = serve.resolve_config(args)
        cfg["memory"]["kv_cache"]["page_size_tokens"] = 16
        cfg.setdefault("autoconfig", {})["vram_expert_ratio"] = ratio
        eng = serve.build_engine(cfg, shape, ckpt, args)
        return shape, eng

    prompt = [(7 * i + 3) % 500 + 4 for i in range(40)]

    def tokens(eng):
        sid = eng.create_sequence()
        out = [eng.prefill(sid, prompt)]
        for _ in range(6):
            out.append(eng.decode([sid], [out[-1]])[0])
        return out

    shape, full = boot(1.0)
    assert full.model.streamer is None
    ref = tokens(full)
    del full
    torch.cuda.empty_cache()
    shape, eng = boot(0.5)
    st = eng.model.streamer
    e_total = shape.n_routed + shape.n_shared
    assert st is not None and not eng.use_graph and st.weighted
    assert all(l["arena"].n_slots == max(shape.top_k + shape.n_shared, e_total // 2) for l in st.layers.values()) and len(st.layers) == shape.n_moe_layers()
    assert tokens(eng) == ref
    s = st.summary()
    assert s["misses"] > 0 and s["bytes_h2d"] > 0


@pytest.mark.parametrize("name,kv", [("tiny-mla-moe", "bf16"), ("tiny-glm5-next", "fp8"), ("tiny-deepseek-v32", "fp8")])
def test_solver_sizing_agrees_with_the_booted_engine(name, kv):
    """The cross-check table of the autoconfig solver against a real engine: KV bytes per token, recurrent state per sequence and
    the page count agree exactly, expert slot and resident weight bytes are never under-estimated."""
    from layerstorm_b200.autoconfig.enginecheck import render, run_checks
    from layerstorm_b200.models.config import get_preset
    from layerstorm_b200.models.device_model import DeviceModel
    from layerstorm_b200.models.weights import init_weights
    from layerstorm_b200.runtime.engine import Engine
    cfg = get_preset(name)
    m = DeviceModel.from_state_dict(cfg, init_weights(cfg, 0), "cuda", kv_fmt=kv, page=16)
    eng = Engine(m, max_seqs=3, max_ctx=256, prefill_chunk=32, max_batch=1)
    res = run_checks(eng)
    table = render(res)
    by = {r.name: r for r in res}
    assert not [r for r in res if r.status == "FAIL"], table
    assert by["kv_bytes_per_token"].status == "ok" and by["kv_pages"].status == "ok", table
    assert by["recurrent_state_bytes_per_sequence"].status == ("ok" if any(cfg.is_kda_layer(i) for i in range(cfg.n_layers)) else "unchecked"), table


def test_continuous_batching_on_the_gpu_engine_matches_sequential_serving():
    """Four concurrent greedy requests through the batched serving loop on the GPU engine (batched decode steps under CUDA graphs,
    one per batch size) produce the tokens of the same requests served one at a time."""
    from layerstorm_b200.serving.orchestrator import InferenceRequest, Orchestrator, SamplingParams
    cfg, eng = _engine("tiny-glm5-next")
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(4, cfg.vocab, (n,), generator=g).tolist() for n in (20, 45, 33, 70)]
    gens = [9, 4, 12, 6]

    def serve(max_batch):
        orch = Orchestrator(eng, eos_token_ids=[], max_batch=max_batch, prefill_slice_tokens=16)      # prompts join in several slices
        reqs = [InferenceRequest(f"b{max_batch}-{i}", list(p), SamplingParams(max_tokens=n, ignore_eos=True)) for i, (p, n) in enumerate(zip(prompts, gens))]
        for r in reqs:
            orch.submit_request(r)
        for _ in range(200):
            if not orch.step():
                break
        assert all(r.done.is_set() and r.error is None for r in reqs), [r.error for r in reqs]
        orch.prefix.clear()
        return [list(r.output_ids) for r in reqs], orch

    want, _ = serve(1)
    got, orch = serve(4)
    assert got == want
    assert 0 < orch.batched_steps < sum(gens) - len(gens)


@pytest.mark.parametrize("name,graph", [("tiny-mla-moe", False), ("tiny-mla-moe", True), ("tiny-glm5-next", False)])
def test_aux_hidden_capture_feeds_a_block_draft_that_matches_the_cpu_draft_and_stays_lossless(name, graph):
    """The engine reports the stream entering the aux layers of every committed step (prefill chunks, verify steps with rejected
    rows, decode steps - eager and as a CUDA graph); the block draft's context built from those reports equals the one built from
    the fp32 reference model's hidden states, so both propose the same block, and greedy speculation with the block draft reproduces
    plain greedy decoding."""
    from layerstorm_b200.models.config import get_preset
    from layerstorm_b200.models.device_model import DeviceModel
    from layerstorm_b200.models.reference import Oracle
    from layerstorm_b200.models.weights import init_weights
    from layerstorm_b200.runtime.engine import Engine
    from layerstorm_b200.speculation import dspark as dsp
    cfg = get_preset(name)
    m = DeviceModel.from_state_dict(cfg, init_weights(cfg, 3), "cuda", kv_fmt="bf16", page=16, expert_quant="bf16", dense_quant="bf16")
    oracle = Oracle(cfg, m.effective_state_dict())
    prompt = torch.randint(0, cfg.vocab, (27,), generator=torch.Generator().manual_seed(4)).tolist()

    plain = Engine(m, max_seqs=2, max_ctx=128, prefill_chunk=8, max_batch=1, use_graph=False)
    s0 = plain.create_sequence()
    want = [plain.prefill(s0, prompt)]
    for _ in range(11):
        want.append(plain.decode([s0], [want[-1]])[0])
    plain.free_sequence(s0)

    dc = dsp.draft_config_for_target(cfg.hidden, cfg.vocab, cfg.n_layers, layers=2, head_dim=16, block_size=5, markov_rank=8, n_aux=2)
    tens = dsp.random_dspark_tensors(dc, 1)
    eng = Engine(m, max_seqs=3, max_ctx=128, prefill_chunk=8, max_batch=1, use_graph=graph)
    dev = dsp.DeviceDsparkDraft(eng, dsp.DsparkBackbone(dc, tens, "cuda", torch.float32, ctx_capacity=128), {"speculative_tokens": 4})
    ref = dsp.DsparkDraft(dsp.DsparkBackbone(dc, tens, "cpu", torch.float32, ctx_capacity=128), dsp.oracle_aux_provider(oracle, dc.aux_hidden_state_layer_ids),
                          {"speculative_tokens": 4})
    seen = []
    inner = dev.on_rows
    dev.on_rows = lambda sid, pos0, aux, toks: (seen.append((pos0, aux.float().cpu().clone())), inner(sid, pos0, aux, toks))[1]
    sid = eng.create_sequence()
    tok = eng.prefill(sid, prompt)
    assert tok == want[0] and [p for p, _ in seen] == [0, 8, 16, 24]
    aux_ref = dsp.oracle_aux_provider(oracle, dc.aux_hidden_state_layer_ids)(prompt, 0)
    got_aux = torch.cat([a for _, a in seen])
    assert got_aux.shape == aux_ref.shape and float((got_aux - aux_ref).abs().max() / aux_ref.abs().max()) < 3e-2
    got, ctx, rounds = [tok], prompt + [tok], 0
    while len(got) < 12:
        d = dev.propose(ctx, 4)
        assert len(d) == 4
        c = dev.ctx[sid]
        rc_ok = ref._follow(ctx[:-1])
        assert rc_ok and c.length == ref.ctx.length == len(ctx) - 1
        kd, kr = c.k[:, : c.length].float().cpu(), ref.ctx.k[:, : c.length]
        assert float((kd - kr).abs().max() / kr.abs().max()) < 5e-2                  # bf16 hidden states against the fp32 model's
        if rounds % 3 == 2:
            tok = eng.decode([sid], [tok])[0]
            new = [tok]
        else:
            n_acc, nxt = eng.verify_greedy(sid, tok, d)                               # random draft: mostly rejected rows, overwritten next step
            new = d[:n_acc] + [nxt]
            tok = nxt
        rounds += 1
        got += new
        ctx += new
    assert got[:12] == want[:12]
    # a fork shares the parent's rows; freeing returns the context
    child = eng.fork_sequence(sid)
    assert dev.propose(ctx, 3) != [] and child in dev.ctx and dev.ctx[child].length == dev.ctx[sid].length
    eng.free_sequence(child)
    assert child not in dev.ctx and len(dev._spare) == 1


@pytest.mark.parametrize("fmt", ["bf16", "fp8_e4m3", "nvfp4"])
def test_block_draft_on_the_frameworks_own_gemm_kernels(fmt):
    """The draft's matrices stored as bf16 / FP8 / NVFP4 and applied by the weight-streaming kernels (a block's few rows) and the
    tcgen05 GEMMs (a context chunk's many rows): context keys and block logits against the fp32 tensor code over the de-quantised
    weights."""
    from layerstorm_b200.speculation import dspark as dsp
    dc = dsp.draft_config_for_target(256, 1024, 4, layers=2, head_dim=64, inter=512, block_size=8, markov_rank=16, n_aux=2)
    tens = dsp.random_dspark_tensors(dc, 5)
    dev = dsp.DsparkBackbone(dc, tens, "cuda", ctx_capacity=128, kernels=fmt)
    ref = dsp.DsparkBackbone(dc, dev.effective_tensors(), "cpu", torch.float32, ctx_capacity=128)
    if fmt == "bf16":
        assert all(torch.equal(v.float(), tens[k].float()) for k, v in dev.effective_tensors().items() if v.is_floating_point())
    else:
        assert dev.weight_bytes() < 0.8 * dsp.DsparkBackbone(dc, tens, "cuda", torch.bfloat16, ctx_capacity=16).weight_bytes()
    aux = torch.randn(43, 512, generator=torch.Generator().manual_seed(6)).to(torch.bfloat16)
    cd, cr = dev.new_context(), ref.new_context()
    for a, b in ((0, 5), (5, 24), (24, 43)):                       # 5 rows: streaming kernels; 19 rows: tensor-core GEMMs
        assert dev.ingest(cd, aux[a:b].cuda(), a) and ref.ingest(cr, aux[a:b].float(), a)
    kd, kr = cd.k[:, :43].float().cpu(), cr.k[:, :43]
    vd, vr = cd.v[:, :43].float().cpu(), cr.v[:, :43]
    assert float((kd - kr).abs().max() / kr.abs().max()) < 3e-2 and float((vd - vr).abs().max() / vr.abs().max()) < 3e-2
    for n in (7, 3, 1):                                            # 8, 4 and 2 rows
        ld, hd = dev.run_block(cd, 77, 43, n)
        lr, hr = ref.run_block(cr, 77, 43, n)
        assert ld.dtype == torch.float32 and float((ld.cpu() - lr).abs().max() / lr.abs().max()) < 4e-2
        assert float((hd.float().cpu() - hr).abs().max() / hr.abs().max()) < 4e-2
    ids, conf = dev.draft(cd, 77, 43, 7)
    assert len(ids) == 7 and len(conf) == 7 and all(0 <= t < 1024 for t in ids)
