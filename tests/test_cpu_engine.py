"""The CPU plumbing configuration: tiny MLA-MoE, 64-token random prompt, 32 greedy tokens - on the fp32 reference and on the
native CPU expert kernels (same tokens), and through the orchestrator."""
import torch

from layerstorm_b200.models.config import get_preset
from layerstorm_b200.models.reference import Oracle
from layerstorm_b200.models.weights import init_weights
from layerstorm_b200.runtime.cpu_engine import CpuEngine, cpu_plumbing_run
from layerstorm_b200.serving.orchestrator import InferenceRequest, Orchestrator, SamplingParams


def test_cpu_plumbing_native_experts_match_reference():
    a, _, tps_a = cpu_plumbing_run(native_experts=False, prompt_len=24, new_tokens=8)
    b, _, tps_b = cpu_plumbing_run(native_experts=True, prompt_len=24, new_tokens=8)
    assert a == b and len(a) == 8 and tps_a > 0 and tps_b > 0
    cfg = get_preset("tiny-mla-moe")
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, cfg.vocab, (24,), generator=g).tolist()
    assert Oracle(cfg, init_weights(cfg, 0)).greedy(prompt, 8) == a


def test_cpu_engine_quantised_experts_and_engine_api():
    cfg = get_preset("tiny-mla-moe")
    w = init_weights(cfg, 1)
    eng = CpuEngine(cfg, w, native_experts=True, expert_quant="nvfp4")
    ref = CpuEngine(cfg, w, native_experts=False)
    prompt = list(range(3, 19))
    s1, s2 = eng.create_sequence(), ref.create_sequence()
    n1, l1 = eng.prefill(s1, prompt, want_logits=True)
    n2, l2 = ref.prefill(s2, prompt, want_logits=True)
    assert float((l1 - l2).abs().max() / l2.abs().max()) < 0.15          # 4-bit experts vs fp32 experts
    rows = eng.forward_rows(s1, [5, 6, 7], commit=False)
    assert rows.shape == (3, cfg.vocab) and eng.seq_len(s1) == 16
    child = eng.fork_sequence(s1, 8)
    assert eng.seq_len(child) == 8
    eng.rewind(s1, 10)
    assert eng.seq_len(s1) == 10
    eng.free_sequence(child)


def test_orchestrator_on_cpu_engine():
    cfg = get_preset("tiny-mla-moe")
    eng = CpuEngine(cfg, init_weights(cfg, 2), native_experts=True)
    orch = Orchestrator(eng)
    req = InferenceRequest("r", list(range(10, 22)), SamplingParams(max_tokens=5, ignore_eos=True))
    orch.submit_request(req)
    orch.step()
    assert len(req.output_ids) == 5 and req.finish_reason == "length"


def test_self_speculative_draft_is_lossless_on_the_cpu_engine():
    from layerstorm_b200.speculation.self_draft import SelfSpeculativeDraft
    cfg = get_preset("tiny-mla-moe")
    w = init_weights(cfg, 3)
    prompt = list(range(7, 31))
    plain = CpuEngine(cfg, w, native_experts=False)
    req0 = InferenceRequest("p", prompt, SamplingParams(max_tokens=12, ignore_eos=True))
    o0 = Orchestrator(plain)
    o0.submit_request(req0)
    assert o0.step() and req0.error is None
    eng = CpuEngine(cfg, w, native_experts=False)
    draft = SelfSpeculativeDraft(eng, {"draft_expert_count": 2, "adaptive_exit_enabled": False}, max_gamma=3)
    assert draft.engine.cfg.top_k == 2 and eng.cfg.top_k == cfg.top_k and draft.engine.model.w is eng.model.w      # same weights, fewer experts
    assert abs(draft.expert_fraction - 2 / cfg.top_k) < 1e-9
    orch = Orchestrator(eng, draft=draft, speculation_depth=3)
    req = InferenceRequest("s", prompt, SamplingParams(max_tokens=12, ignore_eos=True))
    orch.submit_request(req)
    assert orch.step() and req.error is None
    assert req.output_ids == req0.output_ids                     # verification by the full model: same tokens as plain greedy
    assert req.stats.spec_rounds > 0 and draft.plan.steps > 0 and draft.failures == 0
    assert 0.0 <= draft.plan.acceptance_rate <= 1.0


def test_serve_builds_model_drafts_on_the_test_engine():
    from layerstorm_b200.cli import serve
    from layerstorm_b200.speculation.model_draft import EngineDraft
    args = serve.build_parser().parse_args(["--model", "tiny-mla-moe", "--test-engine", "--tokenizer-mode", "byte", "--speculation-depth", "4"])
    cfg, shape, ckpt, _ = serve.resolve_config(args)
    cfg["speculation"]["enabled"], cfg["speculation"]["method"] = True, "dspark"
    eng = serve.build_engine(cfg, shape, ckpt, args)
    _, orch = serve.build_server(cfg, shape, ckpt, eng, args)
    assert isinstance(orch.draft, EngineDraft) and orch.gamma == 4
    req = InferenceRequest("d", list(range(5, 40)), SamplingParams(max_tokens=10, ignore_eos=True))
    orch.submit_request(req)
    assert orch.step() and req.error is None and len(req.output_ids) == 10 and req.stats.spec_accepted > 0
    # the null engine cannot draft for itself: self_speculative degrades to plain decoding with a warning
    cfg["speculation"]["method"] = "self_speculative"
    _, orch2 = serve.build_server(cfg, shape, ckpt, serve.build_engine(cfg, shape, ckpt, args), args)
    assert orch2.draft is None and orch2.gamma == 0


def test_mtp_blocks_and_lossless_mtp_speculation():
    import dataclasses
    from layerstorm_b200.models.mtp import mtp_block, mtp_draft_tokens
    from layerstorm_b200.speculation.mtp_draft import MtpDraft
    base = get_preset("tiny-mla-moe")
    cfg = dataclasses.replace(base, n_mtp=1)
    w = init_weights(cfg, 5)
    w0 = init_weights(base, 5)
    assert all(torch.equal(w[k], w0[k]) for k in w0) and f"layers.{cfg.n_layers}.mtp.eh_proj" in w        # main weights unchanged by the extra blocks
    eng = CpuEngine(cfg, w, native_experts=False)
    orc = eng.model
    ids = list(range(9, 33))
    logits, hidden = orc.forward(torch.tensor(ids), return_hidden=True)
    assert hidden.shape == (len(ids), cfg.hidden) and torch.equal(logits, orc.forward(torch.tensor(ids)))
    # causality of the block: position i does not depend on later positions
    la, ha = mtp_block(orc, 0, hidden[:-1], ids[1:])
    lb, hb = mtp_block(orc, 0, hidden[:10], ids[1:11])
    assert torch.allclose(la[:10], lb, atol=1e-5) and torch.allclose(ha[:10], hb, atol=1e-5)
    toks, conf = mtp_draft_tokens(orc, ids, 3)                     # one block, three depths: cyclic reuse
    assert len(toks) == 3 and all(0 <= t < cfg.vocab for t in toks) and all(0 < c <= 1 for c in conf)
    assert mtp_draft_tokens(orc, ids, 3, stop=lambda s, c: True)[0] == toks[:1]
    # through the orchestrator: random MTP weights draft badly, the output must still equal plain greedy decoding
    plain = CpuEngine(cfg, w, native_experts=False)
    r0 = InferenceRequest("p", ids, SamplingParams(max_tokens=8, ignore_eos=True))
    o0 = Orchestrator(plain)
    o0.submit_request(r0)
    assert o0.step() and r0.error is None
    draft = MtpDraft(eng, {"enabled": True, "max_depth": 2, "dynamic_depth": False})
    orch = Orchestrator(eng, draft=draft, speculation_depth=2)
    r1 = InferenceRequest("m", ids, SamplingParams(max_tokens=8, ignore_eos=True))
    orch.submit_request(r1)
    assert orch.step() and r1.error is None
    assert r1.output_ids == r0.output_ids and r1.stats.spec_rounds > 0 and draft.planner.steps > 0
    import pytest
    with pytest.raises(ValueError):
        MtpDraft(CpuEngine(base, w0, native_experts=False), {})


def test_cpu_expert_bench_runs_every_slot_format(capsys):
    """The stand-alone CPU expert benchmark: every device slot format decodes to finite outputs and reports a rate."""
    import json
    from layerstorm_b200.utils import cpu_expert_bench
    assert cpu_expert_bench.main(["--hidden", "256", "--inter", "256", "--tokens", "1,4", "--reps", "2", "--threads", "2"]) == 0
    rep = json.loads(capsys.readouterr().out)
    assert rep["threads"] == 2 and len(rep["rows"]) == 8
    assert {r["format"] for r in rep["rows"]} == {"bf16", "fp8_e4m3", "nvfp4", "gguf_q4_k"}
    assert all(r["finite"] and r["ms"] > 0 and r["gflop_s"] > 0 for r in rep["rows"])
