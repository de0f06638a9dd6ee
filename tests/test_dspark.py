"""DSpark block draft (speculation/dspark.py) on the CPU: checkpoint contract, the non-causal block pass against a per-head reference
written a second way, context bookkeeping (chunks, overwrite, window rotation), the Markov / confidence heads and lossless serving."""
import dataclasses
import json
import math
import os
import struct

import pytest
import torch

from layerstorm_b200.speculation.dspark import (DsparkBackbone, DsparkCheckpointConfig, DsparkDraft, draft_config_for_target, is_dspark_checkpoint,
                                                 load_dspark_checkpoint, oracle_aux_provider, random_dspark_tensors, validate_tensors,
                                                 write_dspark_checkpoint)


def small_cfg(**kw) -> DsparkCheckpointConfig:
    base = dict(block_size=6, speculative_tokens=5, markov_rank=8, enable_confidence_head=True, confidence_head_with_markov=True, draft_vocab_size=97,
                mask_token_id=96, aux_hidden_state_layer_ids=[1, 3], num_hidden_layers=2, hidden_size=32, num_attention_heads=4, num_key_value_heads=2,
                head_dim=8, intermediate_size=48, rms_norm_eps=1e-5, rope_theta=10000.0, vocab_size=97)
    base.update(kw)
    c = DsparkCheckpointConfig(**base)
    c.check()
    return c


def test_checkpoint_roundtrip_and_fail_closed_validation(tmp_path):
    cfg = small_cfg()
    t = random_dspark_tensors(cfg, 1)
    d = str(tmp_path / "draft")
    write_dspark_checkpoint(d, cfg, t)
    assert is_dspark_checkpoint(d) and not is_dspark_checkpoint(str(tmp_path))
    cfg2, t2 = load_dspark_checkpoint(d)
    assert cfg2 == cfg and set(t2) == set(t) and all(torch.equal(t[k], t2[k]) for k in t)
    assert cfg.weight_bytes() == sum(v.numel() * 2 for v in t.values()) and cfg.context_bytes_per_token() == 2 * 2 * 16 * 2
    # the shipped geometry: 7.6 GB of bf16 weights, 80 KB of draft context per token
    big = DsparkCheckpointConfig(draft_vocab_size=154880, mask_token_id=154856, aux_hidden_state_layer_ids=[8, 23, 39, 55, 70], hidden_size=6144,
                                 num_attention_heads=64, num_key_value_heads=64, head_dim=64, intermediate_size=12288, vocab_size=154880,
                                 enable_confidence_head=True, confidence_head_with_markov=True)
    big.check()
    assert len(big.expected_tensors()) == 64 and abs(big.weight_bytes() / 1e9 - 7.61) < 0.02 and big.context_bytes_per_token() == 81920
    for mutate, what in ((lambda x: x.pop("fc.weight"), "missing tensor fc.weight"), (lambda x: x.update(extra=torch.zeros(1)), "unexpected tensor extra"),
                         (lambda x: x.update({"norm.weight": torch.zeros(31)}), "norm.weight: shape"),
                         (lambda x: x.update({"norm.weight": torch.zeros(32, dtype=torch.int32)}), "norm.weight: dtype")):
        bad = dict(t)
        mutate(bad)
        with pytest.raises(ValueError, match=what):
            validate_tensors(cfg, bad)
    j = cfg.to_json()
    j["speculators_model_type"] = "eagle3"
    with pytest.raises(ValueError, match="not a dspark"):
        DsparkCheckpointConfig.from_json(j)
    with pytest.raises(ValueError, match="vanilla"):
        small_cfg(markov_head_type="gated")
    with pytest.raises(ValueError, match="block_size"):
        small_cfg(speculative_tokens=6)
    # a reduced draft vocabulary ships its id map, which must stay inside the target's vocabulary
    red = small_cfg(draft_vocab_size=40)
    tr = random_dspark_tensors(red, 2)
    assert tr["lm_head.weight"].shape == (40, 32) and tr["markov_head.markov_w2.weight"].shape == (40, 8) and tr["markov_head.markov_w1.weight"].shape == (97, 8)
    validate_tensors(red, tr)
    tr["d2t"] = tr["d2t"] + 1000
    with pytest.raises(ValueError, match="outside the target vocabulary"):
        validate_tensors(red, tr)


def reference_block(cfg, t, aux, anchor, n_draft):
    """The block pass written a second way: per-head loops, explicit rotation of each pair, explicit softmax."""
    f = {k: v.double() for k, v in t.items() if v.is_floating_point()}
    H, hd, nh, nkv = cfg.hidden_size, cfg.head_dim, cfg.num_attention_heads, cfg.num_key_value_heads

    def rms(x, w):
        return x / torch.sqrt((x * x).mean(-1, keepdim=True) + cfg.rms_norm_eps) * w

    def rope(vec, pos):
        out = vec.clone()
        for i in range(hd // 2):
            a = pos * cfg.rope_theta ** (-2.0 * i / hd)
            out[i] = vec[i] * math.cos(a) - vec[i + hd // 2] * math.sin(a)
            out[i + hd // 2] = vec[i + hd // 2] * math.cos(a) + vec[i] * math.sin(a)
        return out
    n_ctx = aux.shape[0]
    feat = rms(aux.double() @ f["fc.weight"].T, f["hidden_norm.weight"])
    ids = [anchor] + [cfg.mask_token_id] * n_draft
    nq = len(ids)
    x = f["embed_tokens.weight"][ids]
    for l in range(cfg.num_hidden_layers):
        p = f"layers.{l}."
        h = rms(x, f[p + "input_layernorm.weight"])
        src = torch.cat([feat, h], 0)                                            # context features and block rows share k / v projections
        K = (src @ f[p + "self_attn.k_proj.weight"].T).view(-1, nkv, hd)
        V = (src @ f[p + "self_attn.v_proj.weight"].T).view(-1, nkv, hd)
        Q = (h @ f[p + "self_attn.q_proj.weight"].T).view(nq, nh, hd)
        out = torch.zeros(nq, nh * hd, dtype=torch.double)
        for hh in range(nh):
            g = hh // (nh // nkv)
            ks = torch.stack([rope(rms(K[j, g], f[p + "self_attn.k_norm.weight"]), j) for j in range(n_ctx + nq)])
            for qi in range(nq):
                qv = rope(rms(Q[qi, hh], f[p + "self_attn.q_norm.weight"]), n_ctx + qi)
                sc = (ks @ qv) / math.sqrt(hd)
                pr = torch.exp(sc - sc.max())
                pr = pr / pr.sum()
                out[qi, hh * hd: (hh + 1) * hd] = pr @ V[:, g]
        x = x + out @ f[p + "self_attn.o_proj.weight"].T
        h = rms(x, f[p + "post_attention_layernorm.weight"])
        g_, u_ = h @ f[p + "mlp.gate_proj.weight"].T, h @ f[p + "mlp.up_proj.weight"].T
        x = x + (g_ / (1 + torch.exp(-g_)) * u_) @ f[p + "mlp.down_proj.weight"].T
    hidden = rms(x, f["norm.weight"])
    return hidden @ f["lm_head.weight"].T, hidden


def test_block_pass_matches_a_per_head_reference_and_is_not_causal():
    cfg = small_cfg()
    t = random_dspark_tensors(cfg, 3, dtype=torch.float32)
    bb = DsparkBackbone(cfg, t, "cpu", torch.float32, ctx_capacity=64)
    aux = torch.randn(11, 2 * 32, generator=torch.Generator().manual_seed(4))
    ctx = bb.new_context()
    assert bb.ingest(ctx, aux, 0) and ctx.length == 11
    logits, hidden = bb.run_block(ctx, 17, 11, 4)
    rl, rh = reference_block(cfg, t, aux, 17, 4)
    assert logits.shape == (5, 97) and torch.allclose(logits.double(), rl, atol=2e-4) and torch.allclose(hidden.double(), rh, atol=2e-4)
    # every row sees every other row of the block: a longer block changes the earlier rows (a causal draft would not)
    l5, _ = bb.run_block(ctx, 17, 11, 5)
    assert (l5[:5] - logits).abs().max() > 1e-4
    # ... and every row sees the anchor and the whole context
    assert (bb.run_block(ctx, 18, 11, 4)[0][4] - logits[4]).abs().max() > 1e-4
    aux2 = aux.clone()
    aux2[0] += 1.0
    ctx2 = bb.new_context()
    bb.ingest(ctx2, aux2, 0)
    assert (bb.run_block(ctx2, 17, 11, 4)[0][4] - logits[4]).abs().max() > 1e-5
    # an empty context (the anchor is the first token) is a block of its own
    e = bb.new_context()
    le, _ = bb.run_block(e, 17, 0, 2)
    assert torch.allclose(le.double(), reference_block(cfg, t, aux[:0], 17, 2)[0], atol=2e-4)
    with pytest.raises(ValueError, match="block size"):
        bb.run_block(ctx, 17, 11, 6)
    with pytest.raises(RuntimeError, match="no context"):
        bb.run_block(ctx, 17, 12, 2)


def test_context_ingest_in_chunks_overwrite_after_a_rejection_and_gaps():
    cfg = small_cfg()
    t = random_dspark_tensors(cfg, 5, dtype=torch.float32)
    bb = DsparkBackbone(cfg, t, "cpu", torch.float32, ctx_capacity=64)
    aux = torch.randn(20, 64, generator=torch.Generator().manual_seed(6))
    whole, parts = bb.new_context(), bb.new_context()
    bb.ingest(whole, aux, 0)
    for a, b in ((0, 7), (7, 8), (8, 20)):
        assert bb.ingest(parts, aux[a:b], a)
    assert torch.allclose(whole.k[:, :20], parts.k[:, :20], atol=1e-6) and torch.allclose(whole.v[:, :20], parts.v[:, :20], atol=1e-6)
    # a verify step ran 5 rows of which 2 survived: the next step's rows overwrite the rejected positions in place
    spec = bb.new_context()
    bb.ingest(spec, aux[:12], 0)
    bb.ingest(spec, torch.randn(5, 64), 12)                     # rows of a speculated suffix
    spec.rewind(14)
    assert spec.length == 14
    bb.ingest(spec, aux[14:20], 14)
    ref = bb.new_context()
    bb.ingest(ref, torch.cat([aux[:12], torch.zeros(2, 64), aux[14:20]]), 0)
    assert torch.allclose(spec.k[:, 14:20], ref.k[:, 14:20], atol=1e-6) and torch.allclose(spec.k[:, :12], ref.k[:, :12], atol=1e-6)
    # a gap (rows beyond the frontier) ends drafting for the context instead of attending to stale rows
    gap = bb.new_context()
    bb.ingest(gap, aux[:5], 0)
    assert not bb.ingest(gap, aux[7:9], 7) and not gap.valid
    with pytest.raises(RuntimeError):
        bb.run_block(gap, 3, 5, 2)
    with pytest.raises(ValueError, match="features"):
        bb.ingest(bb.new_context(), torch.zeros(2, 63), 0)


def test_context_window_rotates_and_keeps_the_newest_positions():
    cfg = small_cfg()
    t = random_dspark_tensors(cfg, 7, dtype=torch.float32)
    small = DsparkBackbone(cfg, t, "cpu", torch.float32, ctx_capacity=16)
    large = DsparkBackbone(cfg, t, "cpu", torch.float32, ctx_capacity=256)
    aux = torch.randn(50, 64, generator=torch.Generator().manual_seed(8))
    a, b = small.new_context(), large.new_context()
    large.ingest(b, aux, 0)
    pos = 0
    for n in (10, 5, 3, 9, 1, 1, 1, 12, 8):
        assert small.ingest(a, aux[pos: pos + n], pos)
        pos += n
        assert a.length == pos and a.length - a.base <= 16
        w = a.length - a.base
        assert torch.allclose(a.k[:, :w], b.k[:, a.base: a.length], atol=1e-6) and torch.allclose(a.v[:, :w], b.v[:, a.base: a.length], atol=1e-6)
    assert a.rotations >= 3 and a.base > 0
    # the block over the window = the block over a context that begins at the window's base (positions stay absolute)
    la, _ = small.run_block(a, 5, 50, 3)
    trimmed = large.new_context()
    trimmed.k[:, : 50 - a.base], trimmed.v[:, : 50 - a.base] = b.k[:, a.base: 50], b.v[:, a.base: 50]
    trimmed.base, trimmed.length = a.base, 50
    assert torch.allclose(la, large.run_block(trimmed, 5, 50, 3)[0], atol=1e-5)
    with pytest.raises(RuntimeError, match="no context"):
        small.run_block(a, 5, a.base - 1, 2)                      # an anchor behind the window
    # without rotation a full window ends drafting; a rewind behind the window starts over
    fixed = DsparkBackbone(cfg, t, "cpu", torch.float32, ctx_capacity=16, rotate=False)
    c = fixed.new_context()
    assert fixed.ingest(c, aux[:16], 0) and not fixed.ingest(c, aux[16:18], 16) and not c.valid
    a.rewind(a.base - 1)
    assert a.length == 0 and a.base == 0 and a.valid


def test_markov_chain_vocabulary_map_and_confidence_cut():
    cfg = small_cfg(draft_vocab_size=40)
    t = random_dspark_tensors(cfg, 9, dtype=torch.float32)
    bb = DsparkBackbone(cfg, t, "cpu", torch.float32, ctx_capacity=64)
    ctx = bb.new_context()
    bb.ingest(ctx, torch.randn(9, 64, generator=torch.Generator().manual_seed(10)), 0)
    logits, hidden = bb.run_block(ctx, 33, 9, 5)
    ids, conf = bb.draft(ctx, 33, 9, 5)
    # the chain by hand: each row's logits are corrected by the token chosen for the row before it; draft ids map to target ids
    w1, w2, d2t = t["markov_head.markov_w1.weight"], t["markov_head.markov_w2.weight"], t["d2t"]
    prev, want, feats = 33, [], []
    for k in range(5):
        e = w1[prev]
        feats.append(e)
        did = int(torch.argmax(logits[k + 1] + w2 @ e))
        prev = did + int(d2t[did])
        want.append(prev)
    assert ids == want and all(0 <= x < 97 for x in ids) and len(conf) == 5 and all(0 < c < 1 for c in conf)
    cw, cb = t["confidence_head.proj.weight"][0], float(t["confidence_head.proj.bias"][0])
    assert conf == pytest.approx([float(torch.sigmoid(torch.cat([hidden[k + 1], feats[k]]) @ cw + cb)) for k in range(5)], abs=1e-6)
    # the block is cut where the running product of the survival probabilities falls under the threshold
    prod, keep = 1.0, 0
    for c in conf:
        prod *= c
        if prod < 0.2:
            break
        keep += 1
    assert bb.draft(ctx, 33, 9, 5, confidence_threshold=0.2)[0] == want[:keep] and keep < 5
    # without the Markov feature the confidence head reads the hidden row alone
    plain = small_cfg(confidence_head_with_markov=False)
    tp = random_dspark_tensors(plain, 11, dtype=torch.float32)
    assert tp["confidence_head.proj.weight"].shape == (1, 32)
    bp = DsparkBackbone(plain, tp, "cpu", torch.float32, ctx_capacity=64)
    cp = bp.new_context()
    bp.ingest(cp, torch.randn(4, 64), 0)
    assert len(bp.draft(cp, 3, 4, 3)[1]) == 3


def _target():
    from layerstorm_b200.models.config import get_preset
    from layerstorm_b200.models.weights import init_weights
    from layerstorm_b200.runtime.cpu_engine import CpuEngine
    cfg = get_preset("tiny-mla-moe")
    w = init_weights(cfg, 5)
    return cfg, w, CpuEngine(cfg, w, native_experts=False)


def test_aux_hidden_states_of_the_reference_model():
    cfg, w, eng = _target()
    orc = eng.model
    ids = torch.arange(7, 27)
    cap = {0: None, 2: None, cfg.n_layers: None}
    trace = []
    logits, final = orc.forward(ids, aux=cap, trace=trace, return_hidden=True)
    assert torch.equal(cap[0], w["embed.weight"][ids])                               # what enters layer 0 is the embedding
    assert torch.equal(cap[2], trace[1]) and torch.equal(cap[cfg.n_layers], final)   # what enters layer 2 is what leaves layer 1
    assert torch.equal(logits, orc.forward(ids))
    aux_of = oracle_aux_provider(orc, [1, 2])
    a = aux_of(ids.tolist(), 5)
    assert a.shape == (15, 2 * cfg.hidden) and torch.equal(a[:, cfg.hidden:], trace[1][5:])
    assert torch.equal(oracle_aux_provider(orc, [1], output_of_layer=True)(ids.tolist(), 0), trace[1])
    with pytest.raises(ValueError, match="outside"):
        oracle_aux_provider(orc, [cfg.n_layers + 3])(ids.tolist(), 0)
    # causal target: the features of a position do not depend on later tokens, so a context can be extended piecewise
    assert torch.allclose(aux_of(ids.tolist()[:12], 0), aux_of(ids.tolist(), 0)[:12], atol=1e-5)


def test_hyper_connection_targets_give_the_mean_over_streams():
    from layerstorm_b200.models.config import tiny_glm5_next
    from layerstorm_b200.models.reference import Oracle
    from layerstorm_b200.models.weights import init_weights
    cfg = tiny_glm5_next()
    if not cfg.mhc:
        pytest.skip("the preset has no hyper-connections")
    orc = Oracle(cfg, init_weights(cfg, 3))
    ids = torch.arange(5, 17)
    cap = {0: None, 1: None, cfg.n_layers: None}
    _, final = orc.forward(ids, aux=cap, return_hidden=True)
    assert all(v.shape == (12, cfg.hidden) for v in cap.values())
    assert torch.allclose(cap[0], orc.w["embed.weight"][ids], atol=1e-6)             # n copies of the embedding: their mean is the embedding
    assert torch.equal(cap[cfg.n_layers], final)


def test_draft_source_follows_contexts_and_speculation_stays_lossless():
    from layerstorm_b200.runtime.cpu_engine import CpuEngine
    from layerstorm_b200.serving.orchestrator import InferenceRequest, Orchestrator, SamplingParams
    cfg, w, eng = _target()
    dc = draft_config_for_target(cfg.hidden, cfg.vocab, cfg.n_layers, layers=2, head_dim=16, block_size=5, markov_rank=8, n_aux=2)
    assert dc.aux_hidden_state_layer_ids == sorted(set(dc.aux_hidden_state_layer_ids)) and all(0 < l < cfg.n_layers for l in dc.aux_hidden_state_layer_ids)
    bb = DsparkBackbone(dc, random_dspark_tensors(dc, 1, dtype=torch.float32), "cpu", torch.float32, ctx_capacity=64)
    calls = []
    inner = oracle_aux_provider(eng.model, dc.aux_hidden_state_layer_ids)

    def aux_of(tokens, first):
        calls.append((len(tokens), first))
        return inner(tokens, first)
    draft = DsparkDraft(bb, aux_of, {"speculative_tokens": 4})
    ctx = list(range(9, 30))
    p1 = draft.propose(ctx, 4)
    assert len(p1) == 4 and all(0 <= x < cfg.vocab for x in p1) and calls == [(20, 0)] and draft.ctx.length == 20
    # two tokens accepted: only the new positions are ingested; the same context again needs none
    ctx2 = ctx + p1[:2]
    draft.propose(ctx2, 4)
    assert calls[-1] == (22, 20)
    n = len(calls)
    assert draft.propose(ctx2, 4) == draft.propose(ctx2, 4) and len(calls) == n
    assert len(draft.propose(ctx2, 2)) == 2 and draft.propose(ctx2, 0) == [] and draft.propose([5], 3) == []
    # a context that diverges (another conversation sharing 11 tokens) keeps the shared positions
    other = ctx[:11] + [77, 78, 79]
    draft.propose(other, 3)
    assert calls[-1] == (13, 11) and draft.ctx.tokens == other[:-1]
    # the proposals are a function of the context alone: a fresh source proposes the same
    fresh = DsparkDraft(DsparkBackbone(dc, random_dspark_tensors(dc, 1, dtype=torch.float32), "cpu", torch.float32, ctx_capacity=64), inner, {"speculative_tokens": 4})
    assert fresh.propose(other, 3) == draft.propose(other, 3)
    # serving: whatever the random draft proposes, the tokens are the target's
    prompt = list(range(40, 58))
    r0 = InferenceRequest("plain", prompt, SamplingParams(max_tokens=10, ignore_eos=True))
    o0 = Orchestrator(CpuEngine(cfg, w, native_experts=False))
    o0.submit_request(r0)
    assert o0.step() and r0.error is None
    orch = Orchestrator(eng, draft=draft, speculation_depth=4)
    r1 = InferenceRequest("spec", prompt, SamplingParams(max_tokens=10, ignore_eos=True))
    orch.submit_request(r1)
    assert orch.step() and r1.error is None
    assert r1.output_ids == r0.output_ids and r1.stats.spec_rounds > 0 and draft.proposed > 0 and bb.block_passes > 0
    # a draft that fails (aux source raises) proposes nothing and serving carries on
    def broken(tokens, first):
        raise RuntimeError("aux source gone")
    bad = DsparkDraft(bb, broken, {})
    assert bad.propose(ctx, 4) == [] and bad.failures == 1


def test_a_draft_that_knows_the_target_gets_its_block_accepted():
    """Acceptance end to end: a draft rigged to predict the target's own greedy continuation (its output head reads a one-hot code
    of the position, which the rigged rows carry) has its whole block accepted, so a request needs fewer target steps."""
    from layerstorm_b200.serving.orchestrator import InferenceRequest, Orchestrator, SamplingParams
    cfg, w, eng = _target()
    prompt = list(range(40, 58))
    truth = eng.model.greedy(prompt, 12)

    class Rigged:
        """Stands in for the backbone: proposes the known continuation from the anchor's position on."""
        def __init__(self):
            self.calls = 0

        def propose(self, context, gamma):
            self.calls += 1
            k = len(context) - len(prompt)
            return truth[k: k + gamma]

        def feedback(self, proposed, accepted):
            self.last = (proposed, accepted)
    rig = Rigged()
    orch = Orchestrator(eng, draft=rig, speculation_depth=4)
    r = InferenceRequest("rig", prompt, SamplingParams(max_tokens=12, ignore_eos=True))
    orch.submit_request(r)
    assert orch.step() and r.error is None and r.output_ids == truth
    assert r.stats.spec_rounds <= 4 and r.stats.spec_accepted >= 8


class _ReportingEngine:
    """The part of an engine the device draft source talks to: sequences with committed tokens, and a report of the aux hidden states
    of every committed step (here computed by the reference model)."""

    def __init__(self, cfg, oracle):
        import types
        self.cfg, self.oracle, self.seqs, self.stream, self._ns, self._next = cfg, oracle, {}, None, types.SimpleNamespace, 0

    def enable_aux_capture(self, layer_ids, listener):
        self.aux_of, self.listener = oracle_aux_provider(self.oracle, layer_ids), listener

    def create(self):
        self._next += 1
        self.seqs[self._next] = self._ns(length=0, tokens=[])
        return self._next

    def feed(self, sid, toks):
        s = self.seqs[sid]
        allt = s.tokens + [int(t) for t in toks]
        self.listener.on_rows(sid, s.length, self.aux_of(allt, s.length), toks)
        s.tokens, s.length = allt, len(allt)

    def rewind(self, sid, n):
        s = self.seqs[sid]
        s.tokens, s.length = s.tokens[:n], n
        self.listener.on_rewind(sid, n)

    def fork(self, parent, n):
        c = self.create()
        self.seqs[c] = self._ns(length=n, tokens=list(self.seqs[parent].tokens[:n]))
        self.listener.on_fork(parent, c, n)
        return c

    def free(self, sid):
        self.seqs.pop(sid)
        self.listener.on_free(sid)


def test_device_draft_source_keeps_a_context_per_engine_sequence():
    from layerstorm_b200.speculation.dspark import DeviceDsparkDraft
    cfg, w, cpu = _target()
    dc = draft_config_for_target(cfg.hidden, cfg.vocab, cfg.n_layers, layers=2, head_dim=16, block_size=5, markov_rank=8, n_aux=2)
    tens = random_dspark_tensors(dc, 1, dtype=torch.float32)
    eng = _ReportingEngine(cfg, cpu.model)
    dev = DeviceDsparkDraft(eng, DsparkBackbone(dc, tens, "cpu", torch.float32, ctx_capacity=64), {"speculative_tokens": 4}, max_contexts=2)
    ref = DsparkDraft(DsparkBackbone(dc, tens, "cpu", torch.float32, ctx_capacity=64), oracle_aux_provider(cpu.model, dc.aux_hidden_state_layer_ids), {"speculative_tokens": 4})
    toks = list(range(9, 30))
    a = eng.create()
    eng.feed(a, toks[:8])                                                  # a prompt in two chunks
    eng.feed(a, toks[8:20])
    assert dev.propose(toks, 4) == ref.propose(toks, 4) != []
    # a verify step commits the token and four draft rows; two are rejected and the next step overwrites their positions
    eng.feed(a, [toks[20], 1, 2, 3, 4])
    eng.rewind(a, 23)
    nxt = toks + [1, 2, 50]
    assert dev.ctx[a].length == 23 and dev.propose(nxt, 4) == ref.propose(nxt, 4) != []
    eng.feed(a, [50])
    assert dev.propose(nxt + [51], 3) == ref.propose(nxt + [51], 3)
    # a context the engine does not hold (or that is a step behind) proposes nothing
    assert dev.propose(nxt + [51, 52], 3) == [] and dev.propose(toks[:5], 3) == []
    # a fork continues from the parent's rows without touching them
    b = eng.fork(a, 12)
    eng.feed(b, [70, 71])
    fk = toks[:12] + [70, 71, 72]
    assert dev.propose(fk, 4) == ref.propose(fk, 4) != [] and dev.propose(nxt + [51], 3) == ref.propose(nxt + [51], 3)
    # a third sequence takes the least recently used context: that sequence stops drafting, the others go on
    dev.propose(fk, 2)                                                    # b is now the most recently used
    c = eng.create()
    eng.feed(c, [5, 6, 7])
    assert set(dev.ctx) == {b, c} and dev.propose(nxt + [51], 3) == [] and dev.propose([5, 6, 7, 8], 2) == ref.propose([5, 6, 7, 8], 2) != []
    eng.feed(a, [51])                                                     # rows of a sequence without a context are ignored
    assert a not in dev.ctx
    # freed contexts are reused, not reallocated
    eng.free(b)
    spare = dev._spare[-1]
    d = eng.create()
    eng.feed(d, [9, 9, 9])
    assert dev.ctx[d] is spare and dev.ctx[d].length == 3 and dev.ctx[d].tokens == [9, 9, 9]
    # a draft trained for another target is refused
    other = dataclasses.replace(dc, hidden_size=dc.hidden_size * 2, num_attention_heads=dc.num_attention_heads * 2)
    with pytest.raises(ValueError, match="trained for"):
        DeviceDsparkDraft(eng, DsparkBackbone(other, random_dspark_tensors(other, 1, dtype=torch.float32), "cpu", torch.float32, ctx_capacity=64))


def test_serve_builds_the_block_draft_from_a_checkpoint_or_random_weights(tmp_path):
    import argparse
    from layerstorm_b200.cli.serve import build_block_draft, build_model_draft
    from layerstorm_b200.config.loader import load_config
    from layerstorm_b200.speculation.dspark import DeviceDsparkDraft
    mc, w, cpu = _target()
    eng = _ReportingEngine(mc, cpu.model)
    eng.dev = torch.device("cpu")
    args = argparse.Namespace(speculation_depth=None, test_engine=False)
    dc = draft_config_for_target(mc.hidden, mc.vocab, mc.n_layers, layers=1, head_dim=16, block_size=5, markov_rank=8, n_aux=2)
    d = str(tmp_path / "spec")
    write_dspark_checkpoint(d, dc, random_dspark_tensors(dc, 3))
    cfg = load_config(None, {"speculation.method": "dspark", "speculation.dspark.checkpoint_path": d, "speculation.dspark.speculative_tokens": 3,
                             "speculation.dspark.draft_context_capacity_tokens": 64})
    draft, depth = build_model_draft(cfg, mc, eng, args)
    assert isinstance(draft, DeviceDsparkDraft) and depth == 3 and draft.bb.cfg == dc and draft.bb.ctx_capacity == 64
    s = eng.create()
    eng.feed(s, list(range(5, 20)))
    assert len(draft.propose(list(range(5, 21)), depth)) == 3
    # without a checkpoint, aux layer ids in the configuration ask for a random block draft
    cfg2 = load_config(None, {"speculation.method": "dspark", "speculation.dspark.aux_hidden_state_layer_ids": [1, 2], "speculation.dspark.block_size": 4,
                              "speculation.dspark.speculative_tokens": 7}, check=False)      # (the validator wants a checkpoint path)
    eng2 = _ReportingEngine(mc, cpu.model)
    eng2.dev = torch.device("cpu")
    d2, depth2 = build_model_draft(cfg2, mc, eng2, args)
    assert isinstance(d2, DeviceDsparkDraft) and depth2 == 3 and d2.bb.cfg.aux_hidden_state_layer_ids == [1, 2]
    # neither: not a block draft; an engine that cannot report aux hidden states: no block draft, and a block-draft checkpoint is not
    # mistaken for an autoregressive draft model
    assert build_block_draft(load_config(None, {"speculation.method": "dspark"}, check=False), mc, eng, args) is None
    assert build_model_draft(cfg, mc, object(), args) == (None, 0)


def test_scheduler_modes_choose_the_verified_prefix():
    from layerstorm_b200.speculation.dspark import DsparkScheduler
    conf = [0.9, 0.8, 0.5, 0.9, 0.2]
    assert DsparkScheduler({}).depth(conf, 5) == 5                                              # off: the whole block
    st = DsparkScheduler({"confidence_enabled": True, "confidence_threshold": 0.5})            # the head alone means: cut at the threshold
    assert st.mode == "static_threshold" and st.survival(conf, 5) == pytest.approx([0.9, 0.72, 0.36, 0.324, 0.0648]) and st.depth(conf, 5) == 2
    assert DsparkScheduler({"confidence_enabled": True, "scheduler_mode": "static_threshold", "confidence_threshold": 0.3}).depth(conf, 5) == 4
    # throughput: one more row is verified while it raises expected tokens per unit of verify cost
    cheap = DsparkScheduler({"confidence_enabled": True, "scheduler_mode": "throughput", "verify_row_cost": 0.03})
    dear = DsparkScheduler({"confidence_enabled": True, "scheduler_mode": "throughput", "verify_row_cost": 0.4})
    a = cheap.survival(conf, 5)
    ratio = lambda k, rc: (1 + sum(a[:k])) / (1 + rc * k)                                      # noqa: E731
    assert cheap.depth(conf, 5) == max(range(6), key=lambda k: ratio(k, 0.03)) == 4      # the fifth row (survival 0.06) costs more than it brings
    assert dear.depth(conf, 5) == max(range(6), key=lambda k: ratio(k, 0.4)) == 2
    assert dear.depth([0.2, 0.9, 0.9], 3) == 0                                                 # a block that starts badly is not worth a wide step
    # temperatures reshape each conditional probability on the logit before the product
    hot = DsparkScheduler({"confidence_enabled": True, "confidence_threshold": 0.5, "sts_temperatures": [2.0, 2.0, 2.0, 2.0, 2.0]})
    assert hot.survival([0.9], 1)[0] == pytest.approx(1 / (1 + math.exp(-math.log(9) / 2))) and hot.depth(conf, 5) < st.depth(conf, 5) + 1
    # without a confidence head the running acceptance rate stands in: a_j = p^j
    px = DsparkScheduler({"scheduler_mode": "static_threshold", "confidence_threshold": 0.3})
    assert px.proxy() == 0.5 and px.depth([], 5) == 1
    for _ in range(12):
        px.record([], 4, 4)
    assert px.proxy() > 0.99 and px.depth([], 5) == 5
    px.record([], 4, 0)
    assert px.proxy() == pytest.approx(0.7, abs=0.01) and px.depth([], 5) == 3                  # 0.7^3 = 0.343 >= 0.3 > 0.7^4
    # a draft that keeps failing is not verified at all - except for one token every few rounds, so that a recovery is noticed
    for _ in range(12):
        px.record([], 1, 0)
    assert px.proxy() < 0.05 and [px.depth([], 5) for _ in range(32)].count(1) == 2 and px.probe_every == 16
    # the trace of (confidences, accepted) rounds feeds the temperature fit: an over-confident head is cooled down
    g = torch.Generator().manual_seed(0)
    over = DsparkScheduler({"confidence_enabled": True, "confidence_trace_capacity": 300})
    for _ in range(400):
        c = (0.80 + 0.15 * torch.rand(3, generator=g)).tolist()
        acc = 0
        for k in range(3):
            if float(torch.rand(1, generator=g)) < 0.55:                                        # the draft is right far less often than it claims
                acc += 1
            else:
                break
        over.record(c, 3, acc)
    assert len(over.trace) == 300 and over.rounds == 400
    temps = over.fit_temperatures()
    assert len(temps) == 3 and temps[0] > 1.5 and over.survival([0.9], 1)[0] < 0.8
    with pytest.raises(ValueError):
        DsparkScheduler({"scheduler_mode": "fastest"})


def test_draft_source_applies_the_scheduler_and_learns_from_feedback():
    cfg, w, eng = _target()
    dc = draft_config_for_target(cfg.hidden, cfg.vocab, cfg.n_layers, layers=1, head_dim=16, block_size=5, markov_rank=8, n_aux=2)
    bb = DsparkBackbone(dc, random_dspark_tensors(dc, 1, dtype=torch.float32), "cpu", torch.float32, ctx_capacity=64)
    aux_of = oracle_aux_provider(eng.model, dc.aux_hidden_state_layer_ids)
    ctx = list(range(9, 30))
    full = DsparkDraft(bb, aux_of, {"speculative_tokens": 4}).propose(ctx, 4)
    cut = DsparkDraft(bb, aux_of, {"speculative_tokens": 4, "confidence_enabled": True, "confidence_threshold": 0.3})
    got = cut.propose(ctx, 4)
    surv, keep = 1.0, 0
    for c in cut.last_confidences:
        surv *= c
        if surv < 0.3:
            break
        keep += 1
    assert len(cut.last_confidences) == 4 and got == full[:keep] and keep < 4
    cut.feedback(len(got), 0)
    assert cut.sched.rounds == (1 if got else 0) and (not got or cut.sched.trace[-1] == (tuple(cut.last_confidences[: len(got)]), 0))
    # no confidence head in the checkpoint: confidence_enabled falls back to the acceptance proxy instead of failing
    plain_cfg = dataclasses.replace(dc, enable_confidence_head=False, confidence_head_with_markov=False)
    pb = DsparkBackbone(plain_cfg, random_dspark_tensors(plain_cfg, 1, dtype=torch.float32), "cpu", torch.float32, ctx_capacity=64)
    pd = DsparkDraft(pb, aux_of, {"speculative_tokens": 4, "confidence_enabled": True, "scheduler_mode": "static_threshold", "confidence_threshold": 0.2})
    assert not pd.sched.use_head and len(pd.propose(ctx, 4)) == 2                               # 0.5^2 = 0.25 >= 0.2 > 0.5^3
    pd.feedback(2, 0)
    pd.feedback(2, 0)
    assert pd.sched.proxy() == pytest.approx(0.245) and len(pd.propose(ctx, 4)) == 1            # one token clears 0.2, two do not


def test_effective_tensors_are_the_loaded_ones_and_kernels_need_a_gpu():
    cfg = small_cfg(draft_vocab_size=40)
    t = random_dspark_tensors(cfg, 12, dtype=torch.float32)
    bb = DsparkBackbone(cfg, t, "cpu", torch.float32, ctx_capacity=64)
    eff = bb.effective_tensors()
    assert set(eff) == set(t) and all(torch.equal(eff[k].to(t[k].dtype), t[k]) for k in t)
    validate_tensors(cfg, eff)
    assert bb.weight_bytes() == sum(v.numel() * 4 for k, v in t.items() if k.endswith("proj.weight") and "confidence" not in k or k in ("fc.weight", "lm_head.weight", "embed_tokens.weight"))
    with pytest.raises(ValueError, match="GPU"):
        DsparkBackbone(cfg, t, "cpu", kernels="fp8_e4m3")


def test_expert_routing_corpus_records_blocks_verdicts_and_routing(tmp_path, monkeypatch):
    """Serving with the block draft writes what the draft knew (per-layer hidden rows, ids, confidences) and what became of it; the
    reference model supplies the target's routing per position; the join pairs draft row k with the routing at anchor_pos + 1 + k."""
    from layerstorm_b200.serving.orchestrator import InferenceRequest, Orchestrator, SamplingParams
    from layerstorm_b200.speculation import epm_corpus as ec
    cfg, w, eng = _target()
    dc = draft_config_for_target(cfg.hidden, cfg.vocab, cfg.n_layers, layers=2, head_dim=16, block_size=5, markov_rank=8, n_aux=2)
    bb = DsparkBackbone(dc, random_dspark_tensors(dc, 1, dtype=torch.float32), "cpu", torch.float32, ctx_capacity=64)
    draft = DsparkDraft(bb, oracle_aux_provider(eng.model, dc.aux_hidden_state_layer_ids), {"speculative_tokens": 4})
    d = str(tmp_path / "corpus")
    wr = ec.CorpusWriter(d)
    draft.attach_corpus(wr)
    prompt = list(range(40, 58))
    r = InferenceRequest("c", prompt, SamplingParams(max_tokens=9, ignore_eos=True))
    orch = Orchestrator(eng, draft=draft, speculation_depth=4)
    orch.submit_request(r)
    assert orch.step() and r.error is None
    full = prompt + r.output_ids
    ec.record_oracle_routing(wr, eng.model, draft.sequence_no, full, first=len(prompt))
    wr.close()
    blocks, man, routes = ec.read_blocks(d), ec.read_manifest(d), ec.read_routing(d)
    assert len(blocks) == wr.blocks == r.stats.spec_rounds and len(man) == wr.manifest_lines == len(blocks) and len(routes) == len(r.output_ids)
    b0 = blocks[0]
    assert b0["anchor_pos"] == len(prompt) and b0["anchor_token"] == r.output_ids[0] and len(b0["ids"]) == 4 and len(b0["conf"]) == 4
    assert b0["hiddens"].shape == (4, 2, cfg.hidden) and b0["hiddens"].dtype == torch.bfloat16 and float(b0["hiddens"].float().abs().max()) > 0
    assert [b["block"] for b in blocks] == list(range(len(blocks))) and all(b["seq"] == draft.sequence_no for b in blocks)
    # the verdicts tell the story of the request: anchor + accepted tokens + the target's own token per round
    pos = len(prompt)
    for b, m in zip(blocks, man):
        assert m["anchor_pos"] == b["anchor_pos"] == pos and m["committed"] == b["ids"][: m["accepted"]] == full[pos + 1: pos + 1 + m["accepted"]]
        pos += m["accepted"] + 1
    # routing records: every routed layer, logits over all experts, the chosen ones on top
    moe_layers = [i for i in range(cfg.n_layers) if cfg.is_moe_layer(i)]
    r0 = routes[0]
    assert r0["pos"] == len(prompt) and [x["layer"] for x in r0["rows"]] == moe_layers and len(r0["rows"][0]["logits"]) == cfg.n_routed
    assert len(r0["rows"][0]["ids"]) == cfg.top_k and abs(sum(r0["rows"][0]["weights"])) > 0
    ex = ec.join_examples(d)
    assert ex and all(e["features"].shape == (2, cfg.hidden) and set(e["labels"]) == set(moe_layers) for e in ex)
    assert all(e["pos"] == b0["anchor_pos"] + 1 + e["row"] for e in ex if e["seq"] == b0["seq"] and e["pos"] <= b0["anchor_pos"] + 4 and e["row"] < 4 and e["pos"] - e["row"] == b0["anchor_pos"] + 1)
    assert sum(1 for e in ex if not e["accepted"]) <= len(blocks)                              # at most the first rejected row of each block
    cov = ec.previous_position_coverage(d)
    assert 0.0 <= cov["coverage"] <= 1.0 and cov["pairs"] == (len(routes) - 1) * len(moe_layers) * cfg.top_k
    # a record cut off by a crash is ignored, everything before it stands; appending continues the corpus
    with open(os.path.join(d, "blocks.bin"), "ab") as f:
        f.write(struct.pack("<III", ec.BLOCK_MAGIC, ec.VERSION, 65535) + b"abc")              # announces 64 KB, holds 3 bytes
    assert len(ec.read_blocks(d)) == len(blocks)
    # the switch: the environment wins over the configuration, "0" forces it off
    assert ec.effective_dump_dir("/x", {}) == "/x" and ec.effective_dump_dir("/x", {"LS_EPM_DUMP": "0"}) == "" and ec.effective_dump_dir("", {"LS_EPM_DUMP": "/y"}) == "/y"
    # a directory that cannot be written switches the writer off instead of failing the request
    blocked = tmp_path / "file"
    blocked.write_text("x")
    off = ec.CorpusWriter(str(blocked / "sub"))
    assert not off.ok
    off.write_manifest(1, 0, 0, 1, 0, [])
    assert off.manifest_lines == 0


def test_autoconfigure_sizes_a_block_draft_and_carries_its_settings(tmp_path, capsys):
    from layerstorm_b200.cli import autoconfigure
    from layerstorm_b200.models.config import get_preset
    from layerstorm_b200.speculation.dspark import draft_memory_bytes
    # the shipped geometry: 7.6 GB in bf16, about half in FP8, 2.7 GB of contexts for four sequences of 8192 positions
    big = DsparkCheckpointConfig(draft_vocab_size=154880, mask_token_id=154856, aux_hidden_state_layer_ids=[8, 23, 39, 55, 70], hidden_size=6144,
                                 num_attention_heads=64, num_key_value_heads=64, head_dim=64, intermediate_size=12288, vocab_size=154880,
                                 enable_confidence_head=True, confidence_head_with_markov=True)
    m = draft_memory_bytes(big, "bf16")
    assert m["weights"] == big.weight_bytes() and m["contexts"] == 81920 * 8192 * 4 and m["total"] == m["weights"] + m["contexts"]
    f8, f4 = draft_memory_bytes(big, "fp8_e4m3")["weights"], draft_memory_bytes(big, "nvfp4")["weights"]
    assert 0.6 * m["weights"] < f8 < 0.7 * m["weights"] and 0.45 * m["weights"] < f4 < 0.55 * m["weights"]      # the embedding stays bf16
    shape = get_preset("glm-5.3-flash")
    dc = draft_config_for_target(shape.hidden, shape.vocab, shape.n_layers, layers=1, head_dim=64, block_size=8, markov_rank=8, n_aux=2)
    d = str(tmp_path / "draft")
    os.makedirs(d)
    json.dump(dc.to_json(), open(os.path.join(d, "config.json"), "w"))              # sizing reads the configuration only
    out = str(tmp_path / "auto.json")
    assert autoconfigure.main(["--model", "glm-5.3-flash", "--assume-gpus", "1", "--draft-checkpoint", d, "--output", out]) == 0
    cfg = json.load(open(out))
    sp = cfg["speculation"]
    assert sp["enabled"] and sp["method"] == "dspark" and sp["dspark"]["checkpoint_path"] == d and sp["dspark"]["block_size"] == 8
    assert sp["dspark"]["aux_hidden_state_layer_ids"] == dc.aux_hidden_state_layer_ids and sp["dspark"]["speculative_tokens"] == 7
    assert "block draft:" in capsys.readouterr().err
    # a draft trained for another target, or something that is not a dspark checkpoint, is refused with a reason
    other = dataclasses.replace(dc, hidden_size=dc.hidden_size // 2, num_attention_heads=dc.num_attention_heads // 2, num_key_value_heads=dc.num_key_value_heads // 2)
    json.dump(other.to_json(), open(os.path.join(d, "config.json"), "w"))
    assert autoconfigure.main(["--model", "glm-5.3-flash", "--assume-gpus", "1", "--draft-checkpoint", d, "--output", out]) == 2
    assert "trained for hidden" in capsys.readouterr().err
    assert autoconfigure.main(["--model", "glm-5.3-flash", "--assume-gpus", "1", "--draft-checkpoint", str(tmp_path), "--output", out]) == 2
    broken = dataclasses.replace(dc, num_key_value_heads=3)                          # a configuration that contradicts itself
    json.dump(broken.to_json(), open(os.path.join(d, "config.json"), "w"))
    assert autoconfigure.main(["--model", "glm-5.3-flash", "--assume-gpus", "1", "--draft-checkpoint", d, "--output", out]) == 2
    assert "multiple of num_key_value_heads" in capsys.readouterr().err


def test_a_corpus_without_labels_is_labelled_offline_from_its_recorded_contexts(tmp_path):
    from layerstorm_b200.serving.orchestrator import InferenceRequest, Orchestrator, SamplingParams
    from layerstorm_b200.speculation import epm_corpus as ec
    from layerstorm_b200.utils import epm_baselines as eb
    cfg, w, eng = _target()
    dc = draft_config_for_target(cfg.hidden, cfg.vocab, cfg.n_layers, layers=2, head_dim=16, block_size=5, markov_rank=8, n_aux=2)
    bb = DsparkBackbone(dc, random_dspark_tensors(dc, 1, dtype=torch.float32), "cpu", torch.float32, ctx_capacity=64)
    draft = DsparkDraft(bb, oracle_aux_provider(eng.model, dc.aux_hidden_state_layer_ids), {"speculative_tokens": 4})
    d = str(tmp_path / "corpus")
    wr = ec.CorpusWriter(d)
    draft.attach_corpus(wr)
    orch = Orchestrator(eng, draft=draft, speculation_depth=4)
    outs = {}
    for name, prompt in (("a", list(range(40, 58))), ("b", list(range(90, 104)))):
        r = InferenceRequest(name, prompt, SamplingParams(max_tokens=7, ignore_eos=True))
        orch.submit_request(r)
        assert orch.step() and r.error is None
        outs[name] = prompt + r.output_ids
    wr.close()
    assert ec.read_routing(d) == [] and ec.join_examples(d) == []                     # feature side only so far
    seqs = ec.sequences_of(d)
    assert len(seqs) == 2
    for toks, full in zip((seqs[k] for k in sorted(seqs)), (outs["a"], outs["b"])):
        assert toks == full[: len(toks)] and len(toks) >= len(full) - 5                   # everything up to the last block's verdict
    n = ec.label_with_oracle(d, eng.model)
    routes = ec.read_routing(d)
    assert n == len(routes) > 0
    # the labels are what the reference model routes at those positions
    eng.model.route_log = {}
    eng.model.forward(torch.tensor(outs["a"]))
    log_a, eng.model.route_log = eng.model.route_log, None
    first = min(r["pos"] for r in routes if r["seq"] == min(seqs))
    rec = next(r for r in routes if r["seq"] == min(seqs) and r["pos"] == first + 2)
    for row in rec["rows"]:
        assert row["ids"] == log_a[row["layer"]][1][first + 2].tolist()
    ex = ec.join_examples(d)
    assert ex and all(e["features"].shape == (2, cfg.hidden) for e in ex)
    rep = eb.evaluate(d, None, widths=(cfg.top_k,))
    assert rep["sequences"] == 2 and rep["locality_prev"][f"recall@{cfg.top_k}"]["n"] > 0


def test_baselines_command_labels_a_corpus_from_a_checkpoint(tmp_path, capsys):
    from layerstorm_b200.models.checkpoint import export_hf
    from layerstorm_b200.serving.orchestrator import InferenceRequest, Orchestrator, SamplingParams
    from layerstorm_b200.speculation import epm_corpus as ec
    from layerstorm_b200.utils import epm_baselines as eb
    cfg, w, eng = _target()
    ck = str(tmp_path / "ck")
    export_hf(cfg, w, ck)
    dc = draft_config_for_target(cfg.hidden, cfg.vocab, cfg.n_layers, layers=1, head_dim=16, block_size=4, markov_rank=8, n_aux=2)
    draft = DsparkDraft(DsparkBackbone(dc, random_dspark_tensors(dc, 1, dtype=torch.float32), "cpu", torch.float32, ctx_capacity=64),
                        oracle_aux_provider(eng.model, dc.aux_hidden_state_layer_ids), {"speculative_tokens": 3})
    d = str(tmp_path / "corpus")
    draft.attach_corpus(ec.CorpusWriter(d))
    orch = Orchestrator(eng, draft=draft, speculation_depth=3)
    for i, prompt in enumerate((list(range(40, 52)), list(range(70, 84)), list(range(100, 110)))):
        r = InferenceRequest(str(i), prompt, SamplingParams(max_tokens=5, ignore_eos=True))
        orch.submit_request(r)
        assert orch.step() and r.error is None
    draft.corpus.close()
    assert eb.main([d, "--label"]) == 2 and "--label needs --weights" in capsys.readouterr().err
    assert eb.main([d, "--weights", ck, "--label", "--widths", str(cfg.top_k)]) == 0
    cap = capsys.readouterr()
    line = json.loads(cap.out.strip().splitlines()[-1])
    assert "labelled" in cap.err and line["examples"] > 0 and "router_probe" in line and not line["in_sample"]


def test_draft_source_reports_what_it_expects_of_its_last_proposal():
    cfg, w, eng = _target()
    dc = draft_config_for_target(cfg.hidden, cfg.vocab, cfg.n_layers, layers=1, head_dim=16, block_size=5, markov_rank=8, n_aux=2)
    bb = DsparkBackbone(dc, random_dspark_tensors(dc, 1, dtype=torch.float32), "cpu", torch.float32, ctx_capacity=64)
    d = DsparkDraft(bb, oracle_aux_provider(eng.model, dc.aux_hidden_state_layer_ids), {"speculative_tokens": 4, "confidence_enabled": True, "confidence_threshold": 0.0})
    assert d.last_expected_tokens() is None
    ids = d.propose(list(range(9, 30)), 4)
    surv, tot = 1.0, 1.0
    for c in d.last_confidences[: len(ids)]:
        surv *= c
        tot += surv
    assert len(ids) == 4 and d.last_expected_tokens() == pytest.approx(tot) and 1.0 < tot < 5.0


def test_block_draft_bench_runs_on_the_cpu_with_the_small_geometry(capsys):
    from layerstorm_b200.utils import dspark_bench
    assert dspark_bench.geometry("shipped").weight_bytes() > 7e9
    assert dspark_bench.main(["--geometry", "small", "--device", "cpu", "--context", "96", "--chunk", "32", "--rows", "4", "--iters", "3"]) == 0
    rep = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert rep["format"] == "fp32-cpu" and rep["block_rows"] == 4 and rep["ingest_ms"] > 0 and rep["block_ms"] > 0 and rep["draft_ms_with_heads"] > 0
    assert rep["ingest_rows_per_s"] > 0 and rep["weight_sweep_gb_s"] > 0 and rep["context"] == 96
    assert dspark_bench.main(["--geometry", "none"]) == 2 and dspark_bench.main(["--geometry", "small", "--device", "cpu", "--rows", "9"]) == 2
