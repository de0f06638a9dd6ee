"""Hidden-state expert predictors, verification planning, STS calibration and the small speculation policies (CPU only)."""
import numpy as np

from layerstorm_b200.config.loader import load_config
from layerstorm_b200.speculation.hidden_predictors import MoeSpeq, Probe
from layerstorm_b200.speculation.policies import (LayerSkipPolicy, PerformanceObjective, ReasoningMode, SelfSpeculativePlan, ThinkTracker,
                                                   cosine)
from layerstorm_b200.speculation.verify_plan import (adaptive_topk, cumulative_survival_ece, fit_sts_temperatures, plan_verification)

H, E, K = 32, 16, 2


def _router(rng, n_layers):
    return [rng.standard_normal((H, E)).astype(np.float32) for _ in range(n_layers)]


def _drive(pred, routers, layers, steps, rng, drift=0.05):
    for _ in range(steps):
        h = rng.standard_normal(H).astype(np.float32)
        for l in range(len(routers)):
            pred.observe_hidden(l, h)
            if l in layers:
                pred.observe_routing(l, np.argsort(-(h @ routers[l]))[:K])
            h = h + drift * rng.standard_normal(H).astype(np.float32)      # the residual stream changes slowly
        pred.end_step()


def test_moe_speq_learns_next_layer_routing():
    rng = np.random.default_rng(1)
    layers = [1, 2, 3, 4]
    routers = _router(rng, 5)
    p = MoeSpeq(H, E, K, layers, lookahead=2, feat=128, lr=0.5, train_interval=16, train_steps=16, warm_samples=64, confidence_threshold=0.2, seed=3)
    assert set(p.heads) == {(1, 2), (1, 3), (2, 3), (2, 4), (3, 4)}
    p.observe_hidden(1, rng.standard_normal(H))
    assert p.predict(1) == []                                              # cold: no hints
    _drive(p, routers, layers, 600, rng)
    assert p.is_warm(1, 2)
    chance = 2 * K / E
    assert p.recall(1, 2) > chance + 0.3 and p.recall(2, 4) > chance + 0.2
    h = rng.standard_normal(H).astype(np.float32)
    p.observe_hidden(1, h)
    hints = p.predict(1)
    assert hints and all(t in (2, 3) and 0 <= e < E and 0.2 <= c <= 1 for t, e, c in hints)
    truth = set(np.argsort(-(h @ routers[2]))[:K])
    assert truth & {e for t, e, _ in hints if t == 2}


def test_probe_predicts_all_later_layers_from_probe_points():
    rng = np.random.default_rng(2)
    layers = list(range(1, 8))
    routers = _router(rng, 8)
    p = Probe(H, E, K, layers, n_layers=8, probe_points=(0.25, 0.5), feat=128, lr=0.5, train_interval=16, train_steps=16, warm_samples=64, seed=5)
    assert p.probe_layers == [2, 4]
    assert {t for s, t in p.heads if s == 4} == {5, 6, 7} and {t for s, t in p.heads if s == 2} == {3, 4, 5, 6, 7}
    _drive(p, routers, layers, 500, rng, drift=0.02)
    assert p.recall(4, 7) > 2 * K / E + 0.3
    assert p.source_layers() == [2, 4]


def test_adaptive_topk_and_verification_plan():
    w = np.array([0.5, 0.3, 0.1, 0.06, 0.04])
    assert adaptive_topk(w, 0.75, 8) == [0, 1] and adaptive_topk(w, 0.95, 8) == [0, 1, 2, 3] and adaptive_topk(w, 0.95, 2) == [0, 1]
    one = lambda *ids: np.bincount(ids, minlength=8).astype(float)
    gating = {(0, 0): one(1, 2), (0, 1): one(3, 4), (1, 0): one(1, 5), (1, 1): one(3, 6), (2, 0): one(7, 2), (2, 1): one(0, 4)}
    resident = {(0, 1), (0, 2), (1, 3), (1, 4)}
    plan = plan_verification(gating, resident, slot_bytes=10_000_000, bandwidth_gbs=10.0, layer_ms=1.0, threshold=0.99, k_max=2, start_ms=1.0)
    assert plan.transfers == [(0, 5), (1, 6), (0, 7), (1, 0)]              # by first position needed, then layer
    assert plan.required[0] == {(0, 1), (0, 2), (1, 3), (1, 4)}
    # 1 ms per transfer; layer 0 starts at 1 ms, layer 1 at 2 ms: position 1's (0,5)@1ms and (1,6)@2ms arrive in time, position 2's (0,7)@3ms does not
    assert plan.max_depth == 2
    assert plan_verification(gating, resident, 10_000_000, 10.0, 1.0, 0.99, 2, start_ms=0.0).max_depth == 1
    assert plan_verification(gating, resident, 10_000_000, 1000.0, 1.0, 0.99, 2, start_ms=1.0).max_depth == 3


def test_sts_calibrates_overconfident_survival():
    rng = np.random.default_rng(0)
    g, rounds = 4, []
    true_p = np.array([0.85, 0.8, 0.75, 0.7])
    for _ in range(4000):
        p = np.clip(true_p + 0.05 * rng.standard_normal(g), 0.05, 0.95)
        ok = rng.random(g) < p
        accepted = int(np.argmin(ok)) if not ok.all() else g
        raw = 1 / (1 + np.exp(-2.0 * np.log(p / (1 - p))))               # over-confident head: logits doubled
        rounds.append((raw, accepted))
    temps = fit_sts_temperatures(rounds, g)
    assert all(1.4 < t < 2.9 for t in temps), temps                        # recovers the logit scale
    before, after = cumulative_survival_ece(rounds, [1.0] * g), cumulative_survival_ece(rounds, temps)
    assert all(a < b for a, b in zip(after, before)) and max(after) < 0.04


def test_reasoning_mode_and_think_tracker():
    cfg = load_config(None, {"speculation.reasoning_mode.enabled": True})["speculation"]["reasoning_mode"]
    rm, tr = ReasoningMode(cfg), ThinkTracker([7, 8], [9])
    states = [tr.feed(t) for t in [1, 7, 8, 2, 3, 9, 4]]
    assert states == [False, False, True, True, True, False, False]
    ov = rm.overrides(True)
    assert ov.active and rm.depth(3, ov) == 6 and ov.adaptive_topk_threshold == 0.85 and ov.sparse_verification
    off = rm.overrides(False)
    assert not off.active and rm.depth(3, off) == 3
    assert not ReasoningMode({"enabled": False}).overrides(True).active


def test_performance_objective_normalises():
    po = PerformanceObjective(3, 1)
    assert abs(po.latency_weight - 0.75) < 1e-12 and po.latency_dominant and abs(po.score(1.0, 0.0) - 0.75) < 1e-12
    assert PerformanceObjective(0, 0).latency_weight == 0.5
    assert PerformanceObjective.from_config(load_config(None)).latency_weight > 0


def test_layer_skip_policy_gates():
    cfg = {"enabled": True, "threshold": 0.99, "no_skip_first": 2, "no_skip_last": 2, "min_contiguous": 2, "product_window": 1,
           "min_acceptance_rate_to_enable": 0.5, "target_skip_fraction": 0.5}
    pol = LayerSkipPolicy(cfg, 12)
    sim = {l: 0.999 for l in range(12)}
    sim[6] = 0.9
    s = pol.skip_set(sim)
    assert s == {4, 5, 6, 9}                                               # needs 2 similar skippable layers below; 7, 8 broken by layer 6
    assert not ({0, 1, 10, 11} & s)
    assert pol.active(0.6) and not pol.active(0.4)
    pol2 = LayerSkipPolicy(dict(cfg, min_contiguous=1, product_window=3, product_threshold=0.995), 12)
    assert 8 not in pol2.skip_set(sim) and 9 not in pol2.skip_set(sim) and 10 not in pol2.skip_set(sim)
    assert abs(cosine([1, 0], [1, 0]) - 1) < 1e-12 and cosine([0, 0], [1, 0]) == 0.0


def test_self_speculative_plan():
    sp = SelfSpeculativePlan({"draft_expert_count": 1, "draft_confidence_threshold": 0.4}, moe_layers=range(1, 6), n_layers=6, model_top_k=8, max_depth=3)
    plan = sp.plan({3})
    assert [p.experts for p in plan] == [0, 1, 1, 0, 1, 1] and plan[3].skip
    assert abs(sp.expert_fraction(8, {3}) - 4 / 40) < 1e-12
    assert sp.should_continue(1, 0.5) and not sp.should_continue(1, 0.3) and not sp.should_continue(3, 0.9)
    sp.record(3, 2)
    sp.record(3, 1)
    assert abs(sp.acceptance_rate - 0.5) < 1e-12


def test_coverage_depth_truncates_at_the_floor():
    from layerstorm_b200.speculation.verify_plan import coverage_depth
    g = np.zeros((3, 2, 8))
    g[0, 0, [1, 2]] = [0.6, 0.4]; g[0, 1, [3, 4]] = [0.5, 0.5]
    g[1, 0, [1, 5]] = [0.9, 0.1]; g[1, 1, [3, 4]] = [0.5, 0.5]
    g[2, 0, [6, 7]] = [0.5, 0.5]; g[2, 1, [3, 4]] = [0.5, 0.5]
    resident = {(10, 1), (10, 2), (11, 3), (11, 4)}
    rep = coverage_depth(g, resident, moe_layers=[10, 11], floor=0.85, threshold=0.99)
    assert rep.depth == 2 and rep.per_position_mode == [0, 1, 1]
    assert abs(rep.per_position_min[1] - 0.9) < 1e-9 and rep.per_position_min[2] == 0.0
    assert "position 2, layer 10" in rep.truncation_reason
    assert coverage_depth(g, resident | {(10, 6), (10, 7)}, [10, 11], 0.85, 0.99).depth == 3


def test_mtp_planner_cycles_blocks_and_gates_depth():
    from layerstorm_b200.speculation.policies import MtpDraftPlanner
    cfg = load_config(None)["speculation"]["mtp"]
    p = MtpDraftPlanner(dict(cfg, max_depth=5), n_layers=61, n_mtp_layers=2)
    steps = p.plan(first_token=42)
    assert [s.layer for s in steps] == [61, 62, 61, 62, 61] and steps[0].input_token == 42 and steps[1].input_token == -1
    assert len(p.plan(1, depth=2)) == 2
    assert p.should_continue(0, 0.9) and not p.should_continue(0, 0.1) and not p.should_continue(4, 0.99)
    p.record(5, 3)
    assert abs(p.acceptance_rate - 0.6) < 1e-12
    assert MtpDraftPlanner(cfg, 61, 0).plan(1) == []


def test_residual_correction_learns_the_missing_experts():
    from layerstorm_b200.speculation.residual_correction import ResidualCorrection
    rng = np.random.default_rng(0)
    Hh, Ee = 16, 8
    A, B = 0.3 * rng.standard_normal((Hh, Hh)).astype(np.float32), rng.standard_normal((Ee, Hh)).astype(np.float32)
    rc = ResidualCorrection(Hh, Ee, mlp_hidden=48, lr=0.1, train_interval=16, train_steps=32, warm_samples=64, seed=1)
    assert not rc.predict(3, np.zeros(Hh), np.zeros(Ee)).any()                 # cold: zero correction
    for _ in range(1500):
        top1 = rng.standard_normal(Hh).astype(np.float32)
        gate = rng.dirichlet(np.ones(Ee)).astype(np.float32)
        full = top1 + np.tanh(top1 @ A) + gate @ B
        rc.record(3, top1, gate, full)
        rc.end_step()
    assert rc.is_warm(3) and rc.error_reduction(3) > 0.6
    top1, gate = rng.standard_normal((4, Hh)).astype(np.float32), rng.dirichlet(np.ones(Ee), 4).astype(np.float32)
    target = np.tanh(top1 @ A) + gate @ B
    pred = rc.predict(3, top1, gate)
    assert pred.shape == (4, Hh) and ((pred - target) ** 2).sum() < 0.5 * (target ** 2).sum()


def test_online_calibrator_moves_the_self_speculative_draft_with_its_acceptance():
    """Low acceptance: layer skipping goes first, then the draft runs more experts per token; high acceptance: fewer experts first,
    then layer skipping comes back - one step per interval, nothing between the thresholds.  On a real (CPU) engine the draft's
    reduced-expert view is rebuilt with the new count and keeps proposing."""
    from layerstorm_b200.models.config import get_preset
    from layerstorm_b200.models.weights import init_weights, round_weights_bf16
    from layerstorm_b200.runtime.cpu_engine import CpuEngine
    from layerstorm_b200.speculation.online_calibrator import DraftParams, OnlineCalibrator
    from layerstorm_b200.speculation.self_draft import SelfSpeculativeDraft
    cal = OnlineCalibrator({"min_acceptance_rate": 0.3, "target_acceptance_rate": 0.6, "adjustment_interval_tokens": 10, "acceptance_ema_alpha": 1.0},
                           DraftParams(draft_expert_count=2, layer_skip_enabled=True, max_draft_expert_count=4))
    assert not cal.update(4, 0)                                   # 4 of 10 tokens: no decision yet
    assert not cal.update(4, 0)
    assert cal.update(4, 0) and cal.params.layer_skip_enabled is False and cal.params.draft_expert_count == 2      # skipping goes first
    for _ in range(3):
        cal.update(4, 0)
    assert cal.params.draft_expert_count == 3
    for _ in range(6):
        cal.update(4, 0)
    assert cal.params.draft_expert_count == 4                    # capped at the model's own top-k
    for _ in range(3):
        assert not cal.update(4, 2)                               # 0.5 lies between the thresholds: nothing moves
    assert cal.params.draft_expert_count == 4
    for _ in range(12):
        cal.update(4, 4)
    assert cal.params.draft_expert_count == 1 and cal.params.layer_skip_enabled is True and cal.adjustments >= 6
    assert not cal.update(0, 0)

    cfg = get_preset("tiny-mla-moe")
    eng = CpuEngine(cfg, round_weights_bf16(init_weights(cfg, 1)), native_experts=False)
    d = SelfSpeculativeDraft(eng, {"enabled": True, "draft_expert_count": 1}, max_gamma=3,
                             calibration={"min_acceptance_rate": 0.3, "target_acceptance_rate": 0.6, "adjustment_interval_tokens": 6,
                                          "acceptance_ema_alpha": 1.0})
    ctx = [5, 9, 33, 71, 20, 8]
    first = d.propose(ctx, 3)
    assert len(first) == 3 and d.engine.cfg.top_k == 1
    old_engine = d.engine
    d.feedback(3, 0)
    d.feedback(3, 0)                                              # 6 drafted tokens, none accepted -> one more expert per token
    assert d.plan.k == 2 and d.engine is not old_engine and d.engine.cfg.top_k == 2 and d.sid is None
    again = d.propose(ctx, 3)
    assert len(again) == 3                                        # the new view rebuilt its cache from the context
    assert abs(d.expert_fraction - 2 / cfg.top_k) < 1e-9
