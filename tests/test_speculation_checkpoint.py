"""Draft proposers, draft heads, combiner / scorer / calibrator, and the lazy checkpoint readers (CPU)."""
import json
import os

import numpy as np
import pytest
import torch

from layerstorm_b200.models.checkpoint import (LazyCheckpoint, dequant_nvfp4_rowmajor, export_hf, hf_config_dict, open_checkpoint)
from layerstorm_b200.models.config import from_hf_config, get_preset, tiny_deepseek_v32, tiny_glm5_next, tiny_mla_moe
from layerstorm_b200.models.weights import init_weights, round_weights_bf16
from layerstorm_b200.runtime.null_engine import NullEngine
from layerstorm_b200.serving.orchestrator import InferenceRequest, Orchestrator, SamplingParams
from layerstorm_b200.speculation import (ConfidenceHead, DepthCalibrator, DraftCombiner, DraftSource, EngineDraft, IncrementalPromptLookup,
                                         MarkovHead, PromptLookupDraft, UtilityScorer, draft_shape_for, expected_tokens)


# ---------------------------------------------------------------- prompt lookup
def test_prompt_lookup_prefers_longest_then_most_recent_match():
    d = PromptLookupDraft(2, 4, 5)
    ctx = [1, 2, 3, 9, 9, 1, 2, 3, 7, 8, 5, 1, 2, 3]
    assert d.propose(ctx, 4) == [7, 8, 5, 1]                 # most recent earlier "1 2 3" is followed by 7 8 5 1
    assert d.propose([4, 5, 6], 4) == []                     # nothing repeats
    assert d.propose([1, 2, 1, 2], 8) == [1, 2]              # continuation is clipped by the context end
    assert d.propose(ctx, 0) == []
    assert PromptLookupDraft(2, 4, 2).propose(ctx, 4) == [7, 8]


def test_incremental_prompt_lookup_matches_rescan():
    g = torch.Generator().manual_seed(3)
    toks = torch.randint(0, 6, (400,), generator=g).tolist()
    a, b = PromptLookupDraft(2, 4, 5), IncrementalPromptLookup(2, 4, 5)
    for n in range(3, 400, 7):
        assert a.propose(toks[:n], 5) == b.propose(toks[:n], 5), n
    assert b.propose([9, 9, 9, 9], 3) == a.propose([9, 9, 9, 9], 3)      # a different sequence resets the index


# ---------------------------------------------------------------- engine draft
def test_engine_draft_tracks_context_and_is_lossless_in_the_orchestrator():
    target = NullEngine(vocab=97, page=16)
    oracle = NullEngine(vocab=97, page=16)
    draft = EngineDraft(NullEngine(vocab=97, page=16), max_gamma=4)     # same deterministic model => perfect draft
    prompt = [5, 6, 7, 8, 9, 10]
    ref = InferenceRequest("ref", list(prompt), SamplingParams(max_tokens=24, ignore_eos=True))
    o = Orchestrator(oracle)
    o.submit_request(ref); o.step()
    req = InferenceRequest("spec", list(prompt), SamplingParams(max_tokens=24, ignore_eos=True))
    s = Orchestrator(target, draft=draft, speculation_depth=4)
    s.submit_request(req); s.step()
    assert req.output_ids == ref.output_ids
    assert req.stats.spec_rounds > 0 and req.stats.spec_accepted > 0
    # the draft cache followed the context without re-prefilling from scratch
    assert draft.failures == 0 and draft.engine.seq_len(draft.sid) >= len(prompt)


def test_engine_draft_rewinds_on_divergent_context_and_fails_closed():
    e = NullEngine(vocab=50, page=16)
    d = EngineDraft(e, max_gamma=3)
    p1 = d.propose([1, 2, 3, 4], 3)
    assert len(p1) == 3 and e.seq_len(d.sid) == 3
    p2 = d.propose([1, 2, 9, 9, 9], 3)                    # diverges after two tokens
    assert len(p2) == 3 and e.seq_len(d.sid) == 4 and d.fed == [1, 2, 9, 9]
    assert d.propose([1, 2, 3, 4], 3) == p1               # deterministic

    class Broken(NullEngine):
        def decode(self, *a, **k):
            raise RuntimeError("draft device lost")
    b = EngineDraft(Broken(vocab=50, page=16))
    assert b.propose([1, 2, 3], 2) == [] and b.failures == 1 and b.sid is None


def test_draft_shape():
    t = get_preset("glm-5.3-flash")
    d = draft_shape_for(t)
    assert d.n_layers == 2 and d.hidden == t.hidden and d.vocab == t.vocab and d.n_routed == 0 and d.dense_quant == "nvfp4"
    assert d.first_k_dense == 2 and not d.has_indexer and d.layer_types == ["mla", "mla"]


# ---------------------------------------------------------------- heads
def test_markov_chain_and_confidence_cut():
    g = torch.Generator().manual_seed(0)
    V, r, G = 40, 8, 5
    w1, w2 = torch.randn(V, r, generator=g), torch.randn(V, r, generator=g)
    base = torch.randn(G, V, generator=g)
    ids, feats = MarkovHead(w1, w2).chain(base, prev_token=3)
    x = 3
    for k in range(G):
        x = int(torch.argmax(base[k] + w2 @ w1[x]))
        assert ids[k] == x
    assert feats.shape == (G, r) and torch.equal(feats[0], w1[3])
    tie = torch.zeros(1, V)
    assert MarkovHead(torch.zeros(V, r), torch.zeros(V, r)).chain(tie, 0)[0] == [0]          # lowest index on ties
    d2t = torch.arange(V) * 0 + 2
    assert MarkovHead(torch.zeros(V, r), torch.zeros(V, r), d2t=d2t).chain(tie, 0)[0] == [2]  # draft -> target vocabulary
    ch = ConfidenceHead(torch.ones(4 + r) * 0.0, b=2.0)
    conf = ch.survival(torch.zeros(G, 4), feats)
    assert torch.allclose(conf, torch.sigmoid(torch.tensor(2.0)).expand(G))
    assert ConfidenceHead.cut(torch.tensor([0.9, 0.9, 0.5, 0.9]), 0.5) == 2
    assert ConfidenceHead.cut(torch.tensor([0.4]), 0.5) == 0


# ---------------------------------------------------------------- combiner / scorer / calibrator
def test_combiner_picks_by_expected_tokens_per_cost_and_learns():
    class Fixed:
        def __init__(self, out): self.out, self.calls = out, 0
        def propose(self, ctx, g): self.calls += 1; return self.out[:g]
    pl, md = Fixed([]), Fixed([1, 2, 3, 4])
    c = DraftCombiner([DraftSource("prompt_lookup", pl, cost=0.0), DraftSource("model", md, cost=0.1)])
    assert c.propose([0], 4) == [1, 2, 3, 4] and c.last.name == "model"
    pl.out = [7, 7, 7, 7]
    assert c.propose([0], 4) == [7, 7, 7, 7] and md.calls == 1          # the free full-length proposal short-circuits
    a0 = c.last.acceptance
    c.feedback(4, 0)
    assert c.last.acceptance < a0
    assert expected_tokens(0.0, 5) == 1.0 and expected_tokens(0.5, 1) == 1.5
    # the chosen source hears about the outcome itself (its planner / scheduler learns), and a source that knows how far it trusts a
    # proposal is weighed by that instead of its running acceptance rate

    class Sure(Fixed):
        def __init__(self, out, exp): super().__init__(out); self.exp, self.heard = exp, []
        def last_expected_tokens(self): return self.exp
        def feedback(self, p, a): self.heard.append((p, a))
    shy, bold = Sure([1, 2, 3, 4], 1.2), Sure([5, 6], 2.9)
    c2 = DraftCombiner([DraftSource("shy", shy, cost=0.1), DraftSource("bold", bold, cost=0.1)])
    assert c2.propose([0], 4) == [5, 6] and c2.last.name == "bold"                 # two trusted tokens beat four doubtful ones
    c2.feedback(2, 2)
    assert bold.heard == [(2, 2)] and shy.heard == []


def test_utility_scorer_strategies():
    s = UtilityScorer("ema", max_depth=8)
    assert s.best_depth(0.05) == 0                     # hopeless draft: do not speculate
    assert s.best_depth(0.9) > s.best_depth(0.6) > 0
    c = UtilityScorer("cascade", static_depth=3, max_depth=8)
    assert c.choose(0.95) == 4 and c.choose(0.95) == 5  # one step per adjustment
    assert UtilityScorer("fixed", static_depth=2).choose(0.1) == 2


def test_depth_calibrator_moves_towards_target_and_disables():
    c = DepthCalibrator(adjustment_interval_tokens=10, depth=3, ema_alpha=1.0)
    for _ in range(5):
        c.record(3, 3)
    assert c.depth == 4 and c.enabled
    c2 = DepthCalibrator(adjustment_interval_tokens=5, depth=3, ema_alpha=1.0)
    for _ in range(6):
        c2.record(3, 0)
    assert not c2.enabled


# ---------------------------------------------------------------- checkpoints
@pytest.mark.parametrize("make", [tiny_mla_moe, tiny_glm5_next, tiny_deepseek_v32])
def test_hf_directory_roundtrip(make, tmp_path):
    cfg = make()
    w = round_weights_bf16(init_weights(cfg))
    export_hf(cfg, w, str(tmp_path), shard_bytes=2 << 20)
    assert len([f for f in os.listdir(tmp_path) if f.endswith(".safetensors")]) > 1
    cfg2, ck = open_checkpoint(str(tmp_path))
    for f in ("hidden", "n_layers", "layer_types", "hc_mult", "kda_rank", "index_kpool", "n_routed", "scoring", "router_bias"):
        assert getattr(cfg2, f) == getattr(cfg, f), f
    for k, v in w.items():
        assert k in ck, k
        got = ck[k]
        assert got.shape == v.shape and torch.equal(got, v), k
    assert "layers.0.nope" not in ck
    with pytest.raises(KeyError):
        ck["layers.0.nope"]


def test_fp8_and_nvfp4_safetensors_linears_are_dequantised(tmp_path):
    from layerstorm_b200.formats import quant
    from layerstorm_b200.formats.safetensors import write_safetensors
    g = torch.Generator().manual_seed(1)
    w = torch.randn(256, 256, generator=g) * 0.05
    q8, sc = quant.quantize_fp8_block(w)
    # NVFP4 in the row-major group-scale layout of ModelOpt checkpoints
    gs = float(w.abs().max()) / (6.0 * 448.0)
    blk = w.reshape(256, 16, 16)
    sf = quant.e4m3_round(blk.abs().amax(-1) / 6.0 / gs).clamp_min(2 ** -9)
    lut = torch.tensor([0, .5, 1, 1.5, 2, 3, 4, 6])
    scaled = blk / (sf.unsqueeze(-1) * gs)
    idx = (scaled.abs().unsqueeze(-1) - lut).abs().argmin(-1)
    nib = (idx + 8 * (scaled < 0)).to(torch.uint8).reshape(256, 256)
    packed = nib[:, 0::2] | (nib[:, 1::2] << 4)
    write_safetensors(str(tmp_path / "model.safetensors"), {
        "a.weight": q8.view(torch.float8_e4m3fn), "a.weight_scale_inv": sc,
        "b.weight": packed, "b.weight_scale": sf.to(torch.float8_e4m3fn), "b.weight_scale_2": torch.tensor([gs]),
        "c.weight": w.to(torch.bfloat16)})
    from layerstorm_b200.models.checkpoint import SafetensorsSource
    s = SafetensorsSource(str(tmp_path))
    assert torch.allclose(s.load("a"), quant.dequantize_fp8_block(q8, sc))
    assert (s.load("a") - w).abs().max() < 0.02
    b = s.load("b")
    assert torch.equal(b, dequant_nvfp4_rowmajor(packed, sf.to(torch.float8_e4m3fn).view(torch.uint8), gs))
    assert (b - w).abs().mean() < 0.01 and (b - w).abs().max() < 0.06
    assert torch.equal(s.load("c"), w.to(torch.bfloat16).float())


def test_gguf_checkpoint_view(tmp_path):
    from layerstorm_b200.formats.gguf import GgufWriter
    cfg = tiny_mla_moe()
    w = round_weights_bf16(init_weights(cfg))
    gw = GgufWriter()
    gw.meta("general.architecture", "deepseek2")
    f32 = lambda t: t.float().numpy()
    gw.add("token_embd.weight", f32(w["embed.weight"]))
    gw.add("output.weight", f32(w["head.weight"]))
    gw.add("output_norm.weight", f32(w["final_norm.weight"]))
    i = 1
    names = {"attn_norm.weight": "attn_norm.weight", "attn.q_a": "attn_q_a.weight", "attn.kv_a": "attn_kv_a_mqa.weight", "attn.o": "attn_output.weight",
             "moe.router": "ffn_gate_inp.weight", "moe.router_bias": "exp_probs_b.bias"}
    for k, n in names.items():
        if f"layers.{i}.{k}" in w:
            gw.add(f"blk.{i}.{n}", f32(w[f"layers.{i}.{k}"]))
    kb = w[f"layers.{i}.attn.k_b"]                                # [H, dl, dn]
    gw.add(f"blk.{i}.attn_k_b.weight", f32(kb.transpose(1, 2).contiguous()))      # stored [H, dn, dl]
    gw.add(f"blk.{i}.attn_v_b.weight", f32(w[f"layers.{i}.attn.v_b"]))
    for proj in ("gate", "up", "down"):
        stack = torch.stack([w[f"layers.{i}.moe.experts.{e}.{proj}"] for e in range(cfg.n_routed)])
        gw.add(f"blk.{i}.ffn_{proj}_exps.weight", f32(stack), ggml_type=8 if proj != "down" else 0)     # Q8_0 for gate/up
        gw.add(f"blk.{i}.ffn_{proj}_shexp.weight", f32(w[f"layers.{i}.moe.shared.0.{proj}"]))
    path = str(tmp_path / "tiny.gguf")
    gw.write(path)
    _, ck = open_checkpoint(path, cfg)
    for k in ("embed.weight", "head.weight", "final_norm.weight", f"layers.{i}.attn.q_a", f"layers.{i}.attn.kv_a", f"layers.{i}.attn.o",
              f"layers.{i}.attn.k_b", f"layers.{i}.attn.v_b", f"layers.{i}.moe.router", f"layers.{i}.moe.experts.3.down", f"layers.{i}.moe.shared.0.up"):
        assert torch.equal(ck[k], w[k]), k
    q = ck[f"layers.{i}.moe.experts.5.gate"]
    ref = w[f"layers.{i}.moe.experts.5.gate"]
    assert q.shape == ref.shape and (q - ref).abs().max() < ref.abs().max() / 100          # Q8_0 error
    assert f"layers.{i}.mlp.gate" not in ck


def test_gguf_q4k_experts_pass_through_bit_exact(tmp_path):
    """Experts stored as Q4_K reach the device format as the file's own super-blocks (no de-quantise / re-quantise round trip)."""
    from layerstorm_b200.formats import gguf as g
    rows, cols, E = 8, 512, 3
    stack = (torch.randn(E, rows, cols, generator=torch.Generator().manual_seed(1)) * 0.05).numpy()
    gw = g.GgufWriter()
    gw.meta("general.architecture", "deepseek2")
    t = g.GGML_TYPES["Q4_K"]
    gw.add("blk.1.ffn_gate_exps.weight", stack, ggml_type=t)
    gw.add("blk.1.ffn_up_exps.weight", stack, ggml_type=g.GGML_TYPES["Q8_0"])
    gw.add("blk.1.ffn_down_shexp.weight", stack[0], ggml_type=t)
    path = str(tmp_path / "q4k.gguf")
    gw.write(path)
    _, ck = open_checkpoint(path, tiny_mla_moe())
    raw = ck.native_q4k("layers.1.moe.experts.2.gate")
    assert raw is not None and tuple(raw.shape) == (rows, cols // 256 * 144) and raw.dtype == torch.uint8
    want = g.quantize(t, stack[2])                                   # the writer's own quantisation of that expert
    assert bytes(raw.numpy().tobytes()) == bytes(want.tobytes())
    deq = torch.from_numpy(g.dequantize(t, raw.numpy().reshape(-1), rows * cols)).reshape(rows, cols)
    assert torch.equal(deq, ck["layers.1.moe.experts.2.gate"])      # same values as the float view
    assert ck.native_q4k("layers.1.moe.experts.2.up") is None        # Q8_0: float path
    sh = ck.native_q4k("layers.1.moe.shared.0.down")
    assert sh is not None and tuple(sh.shape) == (rows, cols // 256 * 144)
    assert ck.native_q4k("layers.1.attn.q_a") is None
    # the general accessor: every block type the GPU kernels decode (here Q4_K and Q8_0), file-order bytes
    t2, raw2, r2, c2 = ck.native_ggml("layers.1.moe.experts.1.up")
    assert (t2, r2, c2) == (g.GGML_TYPES["Q8_0"], rows, cols)
    assert bytes(raw2.tobytes()) == bytes(g.quantize(t2, stack[1]).tobytes())
    t3, raw3, _, _ = ck.native_ggml("layers.1.moe.experts.2.gate")
    assert t3 == t and bytes(raw3.tobytes()) == bytes(want.tobytes())
    assert ck.native_ggml("layers.1.attn.q_a") is None


def test_mtp_block_weights_roundtrip_through_an_hf_checkpoint(tmp_path):
    import dataclasses
    cfg = dataclasses.replace(tiny_mla_moe(), n_mtp=1)
    w = round_weights_bf16(init_weights(cfg))
    export_hf(cfg, w, str(tmp_path))
    cfg2, ck = open_checkpoint(str(tmp_path))
    assert cfg2.n_mtp == 1
    L = cfg.n_layers
    for k in (f"layers.{L}.mtp.enorm", f"layers.{L}.mtp.hnorm", f"layers.{L}.mtp.eh_proj", f"layers.{L}.mtp.final_norm", f"layers.{L}.attn.q_a",
              f"layers.{L}.attn.k_b", f"layers.{L}.attn_norm.weight", f"layers.{L}.moe.router", f"layers.{L}.moe.experts.2.up"):
        assert torch.equal(ck[k], w[k]), k


def test_engine_draft_stops_at_the_first_low_confidence_token():
    """Confidence-gated drafting against an engine that reports a top-1 probability with every token: the draft ends BEFORE the
    first token below the threshold, the engine is rewound to the context, and engines without the capability draft the full depth."""
    from layerstorm_b200.speculation.model_draft import EngineDraft

    class Eng:
        supports_confidence = True
        has_recurrent_state = False

        def __init__(self, confs):
            self.confs, self.calls, self.len, self.rewound = list(confs), 0, 0, None

        def create_sequence(self):
            return 0

        def free_sequence(self, sid):
            pass

        def prefill(self, sid, toks, want_logits=False):
            self.len += len(toks)

        def decode(self, sids, toks, confidence=False):
            c = self.confs[self.calls]
            self.calls += 1
            self.len += 1
            out = [100 + self.calls]
            return (out, [(c, 0.0)]) if confidence else out

        def rewind(self, sid, n):
            self.rewound, self.len = n, n

    ctx = [1, 2, 3, 4]
    e = Eng([0.9, 0.8, 0.2, 0.9])
    d = EngineDraft(e, max_gamma=4, min_confidence=0.5)
    assert d.propose(ctx, 4) == [101, 102]                 # the third token (0.2) and everything after it is not proposed
    assert e.calls == 3 and e.rewound == len(ctx) - 1 and d.early_stops == 1
    e2 = Eng([0.1] * 4)
    assert EngineDraft(e2, max_gamma=4, min_confidence=0.0).propose(ctx, 4) == [101, 102, 103, 104]
    e3 = Eng([0.1] * 4)
    e3.supports_confidence = False
    assert EngineDraft(e3, max_gamma=4, min_confidence=0.5).propose(ctx, 4) == [101, 102, 103, 104]


def test_quant_skip_list_matches_across_namespaces_and_cross_checks(tmp_path):
    """``modules_to_not_convert`` names module paths, multimodal checkpoints store tensors under a wrapper prefix: both are brought into
    one namespace; a list that matches nothing, an FP8 tensor on the list or a scaled non-FP8 tensor off it stop the load."""
    import json as _json
    from layerstorm_b200.models.checkpoint import QuantSkipList
    sk = QuantSkipList(["model.layers.3.self_attn", "lm_head", "visual", "model.layers.5.mlp.gate"], "fp8")
    assert sk.matches("model.language_model.layers.3.self_attn.kv_b_proj.weight")          # wrapper prefix + prefix entry
    assert sk.matches("model.layers.3.self_attn.q_a_proj.weight_scale_inv")                # role suffix stripped
    assert sk.matches("lm_head.weight") and sk.matches("model.visual.blocks.0.attn.qkv.weight")
    assert sk.matches("model.layers.5.mlp.gate.weight") and not sk.matches("model.layers.5.mlp.gate_proj.weight")   # whole path components only
    assert not sk.matches("model.layers.30.self_attn.o_proj.weight")
    shapes = {"model.language_model.layers.3.self_attn.o_proj.weight": (8, 8), "model.language_model.layers.4.mlp.down_proj.weight": (8, 8),
              "model.language_model.layers.4.mlp.down_proj.weight_scale_inv": (1, 1), "model.language_model.norm.weight": (8,)}
    good = {"model.language_model.layers.3.self_attn.o_proj.weight": "BF16", "model.language_model.layers.4.mlp.down_proj.weight": "F8_E4M3",
            "model.language_model.layers.4.mlp.down_proj.weight_scale_inv": "F32", "model.language_model.norm.weight": "BF16"}
    assert sk.cross_check(good, shapes) == {"entries": 4, "matrices_kept": 1}
    with pytest.raises(ValueError, match="FP8 although"):
        sk.cross_check(dict(good, **{"model.language_model.layers.3.self_attn.o_proj.weight": "F8_E4M3"}), shapes)
    with pytest.raises(ValueError, match="carries a quantisation scale"):
        sk.cross_check(dict(good, **{"model.language_model.layers.4.mlp.down_proj.weight": "BF16"}), shapes)
    with pytest.raises(ValueError, match="matches a tensor"):
        QuantSkipList(["transformer.h.0"], "fp8").cross_check(good, shapes)
    (tmp_path / "config.json").write_text(_json.dumps({"text_config": {"quantization_config": {"quant_method": "fp8", "modules_to_not_convert": ["lm_head"]}}}))
    got = QuantSkipList.from_model_dir(str(tmp_path))
    assert got is not None and got.entries == ["lm_head"] and got.quant_method == "fp8"
    (tmp_path / "config.json").write_text("{}")
    assert QuantSkipList.from_model_dir(str(tmp_path)) is None


def test_hash_layers_route_by_the_token_table_and_survive_both_checkpoint_formats(tmp_path):
    """Hash layers (DeepSeek-V4): the experts of a row are its token id's table row, the weights their unbiased scores.
    Reference: src/compute/kernels/moe/hash_gating.h:1-16; table tensor ffn_gate_tid2eid (I32)."""
    import dataclasses
    from layerstorm_b200.formats.gguf import GGML_TYPES, GgufReader, GgufWriter
    from layerstorm_b200.models.reference import Oracle, route_hash
    cfg = dataclasses.replace(tiny_mla_moe(), num_hash_layers=2)
    hashed = [i for i in range(cfg.n_layers) if cfg.is_hash_layer(i)]
    assert hashed and all(cfg.is_moe_layer(i) and i < 2 for i in hashed)
    w = round_weights_bf16(init_weights(cfg))
    tab = w[f"layers.{hashed[0]}.moe.tid2eid"]
    assert tab.dtype == torch.int32 and tab.shape == (cfg.vocab, cfg.top_k)
    assert all(len(set(r.tolist())) == cfg.top_k for r in tab[:64])                  # distinct experts per token
    # routing: ids are the table rows in table order; out-of-range entries are dropped with weight 0
    logits = torch.randn(3, cfg.n_routed)
    t2 = tab.clone().long()
    t2[5, 1] = cfg.n_routed + 3
    ids, wt = route_hash(cfg, logits, t2, torch.tensor([5, 7, cfg.vocab + 1]))
    assert ids[0].tolist() == [int(t2[5, 0]), -1] + t2[5, 2:].tolist() and wt[0, 1] == 0
    assert ids[1].tolist() == t2[7].tolist() and ids[2].tolist() == [-1] * cfg.top_k and float(wt[2].abs().sum()) == 0
    # the oracle's output depends on the token ids through the table: same hidden rows, other ids -> other experts
    o = Oracle(cfg, w)
    tok = torch.randint(0, cfg.vocab, (6,), generator=torch.Generator().manual_seed(1))
    o.forward(tok)
    sel = o.last_route[0]
    last_hashed = max(hashed)
    if last_hashed == cfg.n_layers - 1:
        assert torch.equal(sel, w[f"layers.{last_hashed}.moe.tid2eid"].long()[tok])
    # HuggingFace directory
    export_hf(cfg, w, str(tmp_path / "hf"))
    cfg2, ck = open_checkpoint(str(tmp_path / "hf"))
    assert cfg2.num_hash_layers == 2
    for i in hashed:
        assert torch.equal(ck[f"layers.{i}.moe.tid2eid"].long(), w[f"layers.{i}.moe.tid2eid"].long())
    assert f"layers.{cfg.n_layers - 1}.moe.tid2eid" not in ck or cfg.is_hash_layer(cfg.n_layers - 1)
    # GGUF: an I32 tensor passes through as integers
    gw = GgufWriter()
    gw.meta("general.architecture", "deepseek4")
    gw.add(f"blk.{hashed[0]}.ffn_gate_tid2eid.weight", tab.numpy(), ggml_type=GGML_TYPES["I32"])
    gw.write(str(tmp_path / "t.gguf"))
    r = GgufReader(str(tmp_path / "t.gguf"))
    got = r.get(f"blk.{hashed[0]}.ffn_gate_tid2eid.weight")
    assert got.dtype == np.int32 and np.array_equal(got, tab.numpy())
    _, ck2 = open_checkpoint(str(tmp_path / "t.gguf"), cfg)
    assert torch.equal(ck2[f"layers.{hashed[0]}.moe.tid2eid"].long(), tab.long())


def test_device_mtp_draft_source_finds_the_sequence_of_a_context():
    """``DeviceMtpDraft`` maps the orchestrator's token list to the engine sequence that holds it (minus the token about to be fed) and
    proposes nothing for a context no sequence holds."""
    from layerstorm_b200.speculation.mtp_draft import DeviceMtpDraft

    class Seq:
        def __init__(self, toks):
            self.tokens, self.length = list(toks), len(toks)

    class Eng:
        class cfg:
            n_layers, n_mtp = 4, 1

        def __init__(self):
            self.seqs = {0: Seq([1, 2, 3]), 1: Seq([5, 6, 7, 8])}
            self.calls, self.on = [], False

        def enable_mtp(self):
            self.on = True

        def mtp_draft(self, sid, tok):
            self.calls.append((sid, tok))
            return [42]

    e = Eng()
    d = DeviceMtpDraft(e, {"enabled": True, "max_depth": 3})
    assert e.on
    assert d.propose([5, 6, 7, 8, 9], 4) == [42] and e.calls == [(1, 9)]
    assert d.propose([9, 9, 9], 2) == [] and d.propose([5, 6, 7, 8, 9], 0) == []
    d.feedback(1, 1)
    assert d.proposed == 1


def test_live_gguf_source_builds_slot_images_from_a_real_file(tmp_path):
    """A GGUF file with stacked expert tensors (gate / up in Q4_K, down in Q6_K, shared expert alike) -> ``LiveGgufExpertSource``:
    the slot image of every expert is its three matrices' file blocks in their device layouts at the slot layout's offsets, zeros
    elsewhere; a layer whose tensors are not all natively readable is not covered.  No GPU involved."""
    import dataclasses
    from layerstorm_b200.formats import gguf as g
    from layerstorm_b200.models.device_model import EXPERT_FMT
    from layerstorm_b200.runtime.live_gguf import LiveGgufExpertSource
    cfg = dataclasses.replace(tiny_mla_moe(), moe_inter=256, n_routed=4, top_k=2)
    H, F, E = cfg.hidden, cfg.moe_inter, cfg.n_routed
    gen = torch.Generator().manual_seed(2)
    gw = g.GgufWriter()
    gw.meta("general.architecture", "deepseek2")
    q4, q6, q8 = g.GGML_TYPES["Q4_K"], g.GGML_TYPES["Q6_K"], g.GGML_TYPES["Q8_0"]
    stacks = {}
    for layer, (tgu, tdn) in {1: (q4, q6), 2: (q8, q4)}.items():
        for proj, shape, t in (("gate", (E, F, H), tgu), ("up", (E, F, H), tgu), ("down", (E, H, F), tdn)):
            x = (torch.randn(*shape, generator=gen) * 0.05).numpy()
            stacks[(layer, proj)] = (x, t)
            gw.add(f"blk.{layer}.ffn_{proj}_exps.weight", x, ggml_type=t)
            gw.add(f"blk.{layer}.ffn_{proj}_shexp.weight", x[0] * 0.5, ggml_type=t)
    # layer 3: the up matrix in fp16 - not natively readable
    for proj, shape, t in (("gate", (E, F, H), q4), ("up", (E, F, H), g.GGML_TYPES["F16"]), ("down", (E, H, F), q4)):
        gw.add(f"blk.3.ffn_{proj}_exps.weight", (torch.randn(*shape, generator=gen) * 0.05).numpy(), ggml_type=t)
    path = str(tmp_path / "live.gguf")
    gw.write(path)
    _, ck = open_checkpoint(path, cfg)
    src = LiveGgufExpertSource(ck, cfg, threads=3)
    ef = src.layout(1)
    assert ef is not None and ef.fmt == EXPERT_FMT["gguf_q4_k"] and ef.fmt_down1 == EXPERT_FMT["gguf_q6_k"] + 1
    assert src.layout(2).fmt == EXPERT_FMT["gguf_q8_0"] and src.layout(3) is None and src.layout(0) is None
    host = torch.full((E + cfg.n_shared, ef.stride), 0xAB, dtype=torch.uint8)
    src.build_layer(1, list(range(E + cfg.n_shared)), host)
    for e in range(E + cfg.n_shared):
        img = host[e].numpy()
        used = np.zeros(ef.stride, dtype=bool)
        for proj, off in (("gate", ef.off_gate), ("up", ef.off_up), ("down", ef.off_down)):
            x, t = stacks[(1, proj)]
            mat = x[e] if e < E else x[0] * 0.5
            want = g.to_device_layout(t, g.quantize(t, mat), mat.shape[0], mat.shape[1]).reshape(-1)
            assert np.array_equal(img[off: off + want.size], want), (e, proj)
            used[off: off + want.size] = True
        assert not img[~used].any()                                   # zero tail and padding
    assert src.bytes_built == (E + cfg.n_shared) * ef.stride
    with pytest.raises(ValueError):
        src.load_into(3, 0, host[0].numpy())


def test_depth_policy_follows_the_acceptance_and_probes_after_switching_off():
    from layerstorm_b200.speculation.combiner import DepthPolicy
    from layerstorm_b200.config.loader import load_config
    sp = load_config(None, {}, check=False)["speculation"]
    pol = DepthPolicy.from_config(sp, max_depth=6)
    assert pol is not None and pol.scorer is not None and pol.calibrator is not None and pol.depth() == 3          # static_depth to begin with
    for _ in range(30):                                   # a draft that is always right: the depth climbs one step per round to the cap
        d = pol.depth()
        pol.record(d, d)
    assert pol.acceptance > 0.95 and pol.depth() == min(6, pol.calibrator.depth) and pol.depth() >= 3
    for _ in range(40):                                   # ... that is always wrong: the depth sinks to plain decoding
        d = pol.depth()
        pol.record(max(d, 1), 0)
    assert pol.acceptance < 0.05
    seq = [pol.depth() for _ in range(32)]
    assert seq.count(0) == 30 and seq.count(1) == 2       # a single-token probe every 16 rounds
    # the calibrator's switch-off lasts for the request it happened in
    pol2 = DepthPolicy.from_config(dict(sp, utility_scorer={"enabled": False}, calibration=dict(sp["calibration"], adjustment_interval_tokens=4)), max_depth=4)
    assert pol2.scorer is None and pol2.depth() == 3
    for _ in range(12):
        pol2.record(3, 0)
    assert not pol2.calibrator.enabled and pol2.depth() == 0
    pol2.begin_request()
    assert pol2.depth() >= 1
    assert DepthPolicy.from_config({"utility_scorer": {"enabled": False}}, 4) is None


def test_orchestrator_asks_the_draft_for_the_policys_depth():
    from layerstorm_b200.runtime.null_engine import NullEngine
    from layerstorm_b200.speculation.combiner import DepthPolicy, UtilityScorer
    asked = []

    class Wrong:
        def propose(self, ctx, g):
            asked.append(g)
            return [3] * g                                 # never what the engine continues with
    eng = NullEngine(vocab=300, max_seqs=4)
    pol = DepthPolicy(UtilityScorer("ema", max_depth=4), None, max_depth=4, alpha=0.5, probe_every=5)
    orch = Orchestrator(eng, eos_token_ids=[1], draft=Wrong(), speculation_depth=4, depth_policy=pol)
    r = InferenceRequest("x", list(range(5, 25)), SamplingParams(max_tokens=30, ignore_eos=True))
    orch.submit_request(r)
    assert orch.step() and r.error is None and len(r.output_ids) == 30
    plain = NullEngine(vocab=300, max_seqs=4)
    o0 = Orchestrator(plain, eos_token_ids=[1])
    r0 = InferenceRequest("y", list(range(5, 25)), SamplingParams(max_tokens=30, ignore_eos=True))
    o0.submit_request(r0)
    assert o0.step() and r0.output_ids == r.output_ids
    # the first rounds ask for several tokens, then the policy gives up and only probes with one
    assert asked[0] >= 2 and asked[-1] == 1 and pol.plain_rounds > 0 and len(asked) < 20 and r.stats.spec_accepted == 0


def test_drafts_are_deeper_inside_a_think_block():
    from layerstorm_b200.runtime.null_engine import NullEngine
    from layerstorm_b200.speculation.policies import ReasoningMode
    asked = []

    class Asks:
        def propose(self, ctx, g):
            asked.append((g, ctx[-1]))
            return [3] * g
    OPEN, CLOSE = [250, 251], [252]
    mode = ReasoningMode({"enabled": True, "aggressive_speculation_depth_multiplier": 2.0})
    eng = NullEngine(vocab=300, max_seqs=4)
    orch = Orchestrator(eng, eos_token_ids=[1], draft=Asks(), speculation_depth=3, reasoning=(mode, OPEN, CLOSE))
    r = InferenceRequest("t", list(range(5, 25)) + OPEN, SamplingParams(max_tokens=12, ignore_eos=True))        # the prompt ends inside a think block
    orch.submit_request(r)
    assert orch.step() and r.error is None and len(r.output_ids) == 12
    assert asked and all(g == 6 for g, _ in asked) and orch.think_rounds == len(asked) and orch._think is None
    # outside a think block, or with the mode off, the configured depth is asked for
    asked.clear()
    r2 = InferenceRequest("u", list(range(5, 25)), SamplingParams(max_tokens=8, ignore_eos=True))
    orch.submit_request(r2)
    assert orch.step() and all(g == 3 for g, _ in asked)
    off = Orchestrator(NullEngine(vocab=300, max_seqs=4), eos_token_ids=[1], draft=Asks(), speculation_depth=3,
                       reasoning=(ReasoningMode({"enabled": False}), OPEN, CLOSE))
    assert off.reasoning is None
    # the tracker itself: open and close markers may be several tokens long
    from layerstorm_b200.speculation.policies import ThinkTracker
    tr = ThinkTracker(OPEN, CLOSE)
    states = [tr.feed(t) for t in [9, 250, 251, 40, 41, 252, 42]]
    assert states == [False, False, True, True, True, False, False] and tr.think_tokens == 3
