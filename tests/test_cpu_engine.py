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
    # the model draft sits behind the free source: prompt lookup proposes where the context repeats itself, the model otherwise
    from layerstorm_b200.speculation.combiner import DraftCombiner
    assert isinstance(orch.draft, DraftCombiner) and [s.name for s in orch.draft.sources] == ["prompt_lookup", "dspark"] and orch.gamma == 4
    assert isinstance(orch.draft.sources[1].proposer, EngineDraft) and orch.draft.sources[1].cost == cfg["speculation"]["draft_combiner"]["dspark_compute_cost"]
    req = InferenceRequest("d", list(range(5, 40)), SamplingParams(max_tokens=10, ignore_eos=True))
    orch.submit_request(req)
    assert orch.step() and req.error is None and len(req.output_ids) == 10 and req.stats.spec_accepted > 0
    assert orch.draft.last is not None and orch.draft.last.name == "dspark"            # nothing repeats in this prompt
    # switched off in the configuration: the model draft alone
    cfg["speculation"]["draft_combiner"]["enabled"] = False
    _, orch1 = serve.build_server(cfg, shape, ckpt, serve.build_engine(cfg, shape, ckpt, args), args)
    assert isinstance(orch1.draft, EngineDraft)
    cfg["speculation"]["draft_combiner"]["enabled"] = True
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


def test_loader_xray_tables_and_fits(tmp_path):
    """The loader's trace analysers: demand-fetch frequency table from a routing trace (cold steps left out, concentration profile),
    least-squares copy cost model from copy batches, eviction weights picked by replaying a grid through the cache simulation."""
    import json
    import numpy as np
    from layerstorm_b200.utils import loader_xray as lx
    from layerstorm_b200.utils.cache_sim import synthetic_trace, write_trace
    tr = synthetic_trace(steps=120, layers=3, n_experts=48, top_k=4, zipf=1.2, stickiness=0.4, seed=3)
    rpath = str(tmp_path / "routing.txt")
    write_trace(rpath, tr)
    out = str(tmp_path / "freq.csv")
    assert lx.main(["freq-table", out, rpath, "--slots", "12", "--skip-steps", "3"]) == 0
    table = lx.read_freq_table(out)
    assert table and all(0 <= l < 3 and 0 <= e < 48 and c > 0 for (l, e), c in table.items())
    counts = lx.fetch_counts([tr], 12, skip_steps=3)
    assert counts == table
    # a bigger cache fetches less; a cache that holds every expert fetches each key at most once (its first use)
    assert sum(lx.fetch_counts([tr], 24).values()) < sum(counts.values())
    assert max(lx.fetch_counts([tr], 48, skip_steps=0).values()) == 1
    conc = lx.concentration(counts)
    assert 0 < conc["top_16"] <= conc["top_64"] <= 1.0
    # copy batches generated from a known model: 40 GB/s and 30 us per batch, small noise
    rng = np.random.default_rng(0)
    fpath = str(tmp_path / "fetch.txt")
    with open(fpath, "w") as fh:
        fh.write("# W step copies bytes device_us\n")
        for i in range(200):
            n = int(rng.integers(1, 9))
            b = n * (21 << 20)
            fh.write(f"W {i} {n} {b} {30.0 + b / 40e3 + rng.normal(0, 2.0):.1f}\n")
    rep = lx.fit_constants(lx.read_fetch_trace(fpath), calib_gbs=55.0)
    assert abs(rep["h2d_gb_s"] - 40.0) < 0.5 and abs(rep["batch_overhead_us"] - 30.0) < 3.0 and rep["r2"] > 0.999
    assert rep["against_calibration"]["scale"] > 1.3                   # the calibration's 55 GB/s was optimistic by 55 / 40
    assert lx.main(["fit-constants", fpath, "--out", str(tmp_path / "c.json")]) == 0 and json.load(open(tmp_path / "c.json"))["batches"] == 200
    # policy fit: never worse than the baselines it reports, and the section it writes is loadable by the native cache
    pol = lx.fit_policy(tr, 12)
    best = max(pol["best_weighted"]["hit_rate"], max(pol["baselines"].values()))
    sec = pol["memory.expert_cache"]
    assert sec["eviction_policy"] in ("impact_weighted_lru", "lru", "lfu") and pol["candidates"] >= 20
    from layerstorm_b200.utils.cache_sim import simulate
    w = [sec.get(k, 0.0) for k in lx.WEIGHT_FIELDS] if sec["eviction_policy"] == "impact_weighted_lru" else None
    assert abs(simulate(tr, 12, sec["eviction_policy"], w)["hit_rate"] - best) < 1e-9


def test_expert_predictor_offline_training_beats_fixed_rankings_on_held_out_sequences(tmp_path):
    """Closed-form ridge fit of the reuse predictor over recorded routing, sequence-level split, recall@m against the fixed
    rankings, bundle round trip into the online predictor and into the cache replay."""
    import json
    import numpy as np
    import pytest
    from layerstorm_b200.speculation.expert_ridge import ExpertRidge
    from layerstorm_b200.utils import expert_predictor_train as ept
    from layerstorm_b200.utils.cache_sim import simulate, synthetic_trace, write_trace
    # five sequences over the same expert popularity (one seed), of different lengths and starting points
    paths = []
    for i in range(5):
        p = str(tmp_path / f"r{i}.txt")
        write_trace(p, synthetic_trace(steps=80 + 7 * i, layers=3, n_experts=40, top_k=4, zipf=1.1, stickiness=0.55, seed=10)[9 * i:])
        paths.append(p)
    out = str(tmp_path / "pred.npz")
    assert ept.main(["--traces", *paths, "--out", out, "--report", str(tmp_path / "rep.json")]) == 0
    rep = json.load(open(tmp_path / "rep.json"))
    assert rep["train_sequences"] == 4 and rep["held_out_sequences"] == 1
    h = rep["held_out"]
    k = str(h["pools"][1])
    assert h["trained"][k] >= max(h["previous_position"][k], h["fast_ema"][k], h["slow_ema_frequency"][k]) - 0.01
    assert h["trained"][k] > h["slow_ema_frequency"][k] + 0.02           # temporal locality is learnt, not only popularity
    # bundle -> online predictor (frozen) -> same scores as the trainer's weights
    r = ExpertRidge(3, 40, 4)
    r.load_weights(out)
    assert r.refresh == 0 and np.allclose(r.w, np.load(out)["w"])
    with pytest.raises(ValueError):
        ExpertRidge(2, 40, 4).load_weights(out)
    assert ept.main(["--traces", paths[-1], "--evaluate", out]) == 0
    # the cache replay takes the bundle for its prefetcher
    from layerstorm_b200.utils.cache_sim import read_trace
    tr = read_trace(paths[-1])
    a = simulate(tr, 10, prefetch_budget=2, predictor_weights=out)
    b = simulate(tr, 10, prefetch_budget=0)
    assert a["prefetched"] > 0 and a["misses"] <= b["misses"]


def test_cpu_engine_runs_hash_layers_through_the_native_expert_kernels():
    """A model whose first MoE layers route by the token-id table: the CPU engine (native expert kernels) gives the reference
    model's tokens; the table, not the router's ranking, picks the experts."""
    import dataclasses
    import torch
    from layerstorm_b200.models.config import get_preset
    from layerstorm_b200.models.reference import Oracle
    from layerstorm_b200.models.weights import init_weights, round_weights_bf16
    from layerstorm_b200.runtime.cpu_engine import CpuEngine
    cfg = dataclasses.replace(get_preset("tiny-mla-moe"), num_hash_layers=3)
    w = round_weights_bf16(init_weights(cfg, 2))
    prompt = torch.randint(0, cfg.vocab, (24,), generator=torch.Generator().manual_seed(3)).tolist()
    ref = Oracle(cfg, w).greedy(prompt, 5)
    eng = CpuEngine(cfg, w, native_experts=True)
    sid = eng.create_sequence()
    tok = eng.prefill(sid, prompt)
    got = [tok]
    for _ in range(4):
        got.append(eng.decode([sid], [got[-1]])[0])
    assert got == ref


def test_performance_objective_sets_the_prefill_slice_of_the_batched_server():
    from layerstorm_b200.cli import serve
    args = serve.build_parser().parse_args(["--model", "tiny-mla-moe", "--test-engine", "--tokenizer-mode", "byte"])
    cfg, shape, ckpt, _ = serve.resolve_config(args)
    chunk = int(cfg["orchestrator"]["prefill_chunk_tokens"])
    assert serve.prefill_slice_factor(cfg) == 4                                       # the default 0.6 / 0.4
    _, orch = serve.build_server(cfg, shape, ckpt, serve.build_engine(cfg, shape, ckpt, args), args)
    assert orch.prefill_slice == 4 * chunk
    cfg["orchestrator"]["performance_objective"] = {"latency_weight": 0.9, "throughput_weight": 0.1}
    _, lat = serve.build_server(cfg, shape, ckpt, serve.build_engine(cfg, shape, ckpt, args), args)
    cfg["orchestrator"]["performance_objective"] = {"latency_weight": 0.2, "throughput_weight": 0.8}
    _, thr = serve.build_server(cfg, shape, ckpt, serve.build_engine(cfg, shape, ckpt, args), args)
    assert lat.prefill_slice == chunk and thr.prefill_slice == 8 * chunk
