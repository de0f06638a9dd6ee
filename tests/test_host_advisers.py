"""Config hot reload, GPU load balancer and prefetch fuser (host-side, CPU only)."""
import json
import os

import numpy as np

from layerstorm_b200.config.hot_reload import ConfigHotReloader, diff_configs
from layerstorm_b200.config.loader import get_path, load_config
from layerstorm_b200.runtime.balancer import GpuLoadBalancer, PrefetchFuser


def _write(path, tree, bump):
    with open(path, "w") as fh:
        json.dump(tree, fh)
    os.utime(path, ns=(bump, bump))          # distinct mtime even on coarse clocks


def test_hot_reload_applies_only_live_fields(tmp_path):
    p = str(tmp_path / "cfg.json")
    _write(p, {}, 1_000_000_000)
    cfg = load_config(p)
    holder = cfg["memory"]["expert_cache"]                       # a component keeps a reference into the tree
    seen = []
    r = ConfigHotReloader(p, cfg, on_apply=seen.append)
    assert r.poll() == []                                        # unchanged file
    _write(p, {"memory": {"expert_cache": {"eviction_policy": "lru"}}, "orchestrator": {"max_batch_size": 7},
               "model": {"use_mmap": False}}, 2_000_000_000)
    applied = r.poll()
    assert {c[0] for c in applied} == {"memory.expert_cache.eviction_policy", "orchestrator.max_batch_size"}
    assert holder["eviction_policy"] == "lru" and get_path(cfg, "orchestrator.max_batch_size") == 7
    assert get_path(cfg, "model.use_mmap") is True               # not live: kept until restart, reported
    assert [c[0] for c in r.ignored] == ["model.use_mmap"]
    assert seen == [applied]
    assert r.poll() == []


def test_hot_reload_keeps_config_on_invalid_file(tmp_path):
    p = str(tmp_path / "cfg.json")
    _write(p, {}, 1_000_000_000)
    cfg = load_config(p)
    before = json.dumps(cfg, sort_keys=True)
    r = ConfigHotReloader(p, cfg)
    with open(p, "w") as fh:
        fh.write("{ not json")
    os.utime(p, ns=(3_000_000_000, 3_000_000_000))
    assert r.poll() == [] and r.last_error
    _write(p, {"orchestrator": {"max_batch_size": -5}}, 4_000_000_000)
    assert r.poll() == [] and r.last_error
    assert json.dumps(cfg, sort_keys=True) == before
    _write(p, {"orchestrator": {"max_batch_size": 3}}, 5_000_000_000)
    assert [c[0] for c in r.poll()] == ["orchestrator.max_batch_size"] and r.last_error is None


def test_diff_configs_lists_changed_leaves():
    a = load_config(None)
    b = load_config(None, {"speculation.mtp.max_depth": 9})
    assert diff_configs(a, b) == [("speculation.mtp.max_depth", get_path(a, "speculation.mtp.max_depth"), 9)]


def test_load_balancer_reduces_the_busiest_gpu():
    rng = np.random.default_rng(0)
    bal = GpuLoadBalancer(n_layers=2, n_experts=16, n_gpus=4, decay=1.0, threshold=1.1, max_moves=8)
    hot = [0, 4, 8, 12]                                          # all on GPU 0 under the default placement
    for _ in range(200):
        bal.observe(0, list(rng.choice(hot, 2, replace=False)) + list(rng.integers(0, 16, 2)))
        bal.observe(1, rng.integers(0, 16, 4))                   # balanced layer
    before = bal.imbalance(0)
    assert before > 1.5 and bal.imbalance(1) < 1.3
    moves = bal.propose()
    assert moves and all(m.layer == 0 and m.src == 0 and m.gain > 0 for m in moves[:1])
    bal.apply(moves)
    assert bal.imbalance(0) < before
    assert bal.gpu_loads(0).sum() == bal.load[0].sum()           # nothing lost
    # no free slot on any target: nothing proposed
    bal2 = GpuLoadBalancer(1, 8, 2, decay=1.0)
    for _ in range(50):
        bal2.observe(0, [0, 2, 4])
    assert bal2.propose(slots_free=[0, 0]) == []
    assert bal2.propose(slots_free=[0, 1])


def test_load_balancer_quiet_when_balanced():
    bal = GpuLoadBalancer(1, 8, 2, decay=1.0)
    for _ in range(10):
        bal.observe(0, range(8))
    assert bal.propose() == []


def test_prefetch_fuser_merges_sources_under_a_budget():
    f = PrefetchFuser(slot_bytes=100, budget_bytes=350)
    sug = {"prescope": [(3, 5, 0.9), (3, 6, 0.2), (3, 9, 0.5)],
           "ridge": [(3, 6, 0.9), (4, 1, 0.8), (3, 7, 1.0)],
           "draft": [(3, 7, 0.5), (3, -1, 1.0)]}
    out = f.fuse(sug, resident={(3, 9)}, in_flight={(4, 1)})
    assert len(out) == 3                                         # budget: 3 slots
    assert [(j, e) for j, e, _ in out] == [(3, 5), (3, 7), (3, 6)]
    s = dict(((j, e), v) for j, e, v in out)
    assert abs(s[(3, 7)] - (1 - (1 - 0.5) * (1 - 0.4))) < 1e-6   # two sources agree: combined as independent evidence
    assert abs(s[(3, 6)] - (1 - (1 - 0.2) * (1 - 0.45))) < 1e-6
    assert PrefetchFuser(100, 0).fuse(sug) == []


def test_expert_cache_weighted_score_and_hysteresis():
    from layerstorm_b200.runtime import native as rt
    ec = rt.ExpertCache(4, 0)
    for e in range(4):
        ec.reserve(0, e)
        ec.mark_ready(0, e)
    section = load_config(None)["memory"]["expert_cache"]
    ec.configure(dict(section, eviction_alpha_recency=0.0, eviction_beta_frequency=1.0, eviction_gamma_routing_weight=0.0))
    ec.set_hysteresis(stages=3, up=2, down=1, window_steps=4, ema=0.25)
    for step in range(16):                                   # expert 0 every step, 1 every other step, 2 once, 3 never
        ec.touch(0, 0, 0.5)
        if step % 2 == 0:
            ec.touch(0, 1, 0.2)
        if step == 3:
            ec.touch(0, 2, 0.9)
        ec.end_step()
    st = [ec.slot_stats(ec.lookup(0, e)) for e in range(4)]
    assert st[0]["frequency"] > st[1]["frequency"] > st[2]["frequency"] > st[3]["frequency"] == 0.0
    assert st[0]["temporal_autocorr"] > 0.9 * st[0]["frequency"] and st[1]["temporal_autocorr"] == 0.0
    assert st[0]["hysteresis"] == 1.0 and st[3]["hysteresis"] == 0.0
    assert ec.pick_victim()[2] == 3                          # frequency only: the never-used expert goes first
    ec.touch(0, 3, 0.1)                                      # most recent now, still the least frequent
    assert ec.pick_victim()[2] == 3
    ec.set_weights("impact_weighted_lru", [1.0, 0, 0, 0, 0, 0, 0])     # hot reload: recency only
    assert ec.pick_victim()[2] == 2
    ec.set_weights("impact_weighted_lru", [0.0, 0, 0, 0, 0, 1.0, 0])   # prefetch score protects an expert the advisers expect
    for e in (0, 1, 3):
        assert ec.set_hint(0, e, prefetch_score=0.5)
    assert ec.pick_victim()[2] == 2
    assert ec.set_hint(0, 2, prefetch_score=0.9) and ec.pick_victim()[2] in (0, 1, 3)
    assert not ec.set_hint(5, 5, 0.1, 0.1)
    # hysteresis: an idle window demotes one stage at a time
    ec.set_weights("impact_weighted_lru", [0, 0, 0, 0, 0, 0, 1.0])
    for _ in range(4):
        ec.end_step()
    assert abs(ec.slot_stats(ec.lookup(0, 0))["hysteresis"] - 2 / 3) < 1e-6


def test_work_queue_orders_and_cancels():
    from layerstorm_b200.runtime.scheduling import DONE, PENDING, READY, RUNNING, WorkQueue
    q = WorkQueue()
    q.insert(("a", 0, "attn"), 1.0)
    q.insert(("a", 1, "moe"), 5.0)
    q.insert(("b", 0, "attn"), 5.0)
    q.insert(("b", 1, "moe"), 9.0, status=PENDING)
    assert q.pop().key == ("a", 1, "moe")                        # highest priority, FIFO among equals; PENDING is not handed out
    assert q.get(("a", 1, "moe")).status == RUNNING
    q.update_priority(("a", 0, "attn"), 7.0)
    assert q.pop().key == ("a", 0, "attn")
    q.update_status(("b", 1, "moe"), READY)
    assert q.pop().key == ("b", 1, "moe")
    q.update_status(("a", 1, "moe"), DONE)
    assert len(q) == 3 and q.cancel_by_request("b") == 2 and len(q) == 1
    assert q.pop() is None and [i.key for i in q.by_status(RUNNING)] == [("a", 0, "attn")]
    q.insert(("c", 0, "x"), 1.0)
    q.insert(("c", 1, "x"), 2.0)
    assert [i.key[1] for i in q.pop_n(5)] == [1, 0]


def test_transfer_planner_budget_dedup_and_zones():
    from layerstorm_b200.runtime.scheduling import Candidate, TransferPlanner, ZONE_STABLE, ZONE_STREAMING
    tp = TransferPlanner(n_gpus=2, expert_bytes=20_000_000, link_gbs=[50.0, 50.0], cycle_budget_us=1000.0, max_inflight_per_gpu=3)
    # 50 GB/s * 1 ms = 50 MB per cycle and GPU: two experts of 20 MB fit
    cands = [Candidate(1, 1, 0, 0.9, needed_in_us=5000), Candidate(1, 2, 0, 0.5), Candidate(1, 3, 0, 0.4), Candidate(1, 4, 0, 0.001),
             Candidate(2, 1, 1, 0.8), Candidate(2, 2, 1, 0.75), Candidate(2, 3, 1, 0.6), Candidate(2, 1, 1, 0.3), Candidate(9, 9, 5, 1.0)]
    plan = tp.plan_transfers(cands, resident={1: {(2, 1)}}, in_flight={1: {(2, 2)}}, transfer_latency_us={0: 400.0})
    got = [(t.gpu, t.layer, t.expert) for t in plan]
    assert got == [(0, 1, 1), (1, 2, 3), (0, 1, 2)]              # resident, in flight, below threshold, bad GPU and over budget are skipped
    assert plan[0].zone == ZONE_STABLE and plan[0].start_delay_us == 4600.0 and plan[2].zone == ZONE_STREAMING and plan[2].start_delay_us == 0.0
    ev = tp.plan_evictions({0: 3, 1: 1}, {0: 1, 1: 4}, victims_of=lambda g, n: [(7, i) for i in range(10)])
    assert ev == {0: [(7, 0), (7, 1)]}


def test_live_eviction_change_reaches_the_engine_through_the_spmd_facade():
    from layerstorm_b200.cli.serve import apply_live_changes
    from layerstorm_b200.runtime.spmd import MIRRORED, SpmdLeader
    calls, sent = [], []

    class Eng:
        def configure_expert_cache(self, section):
            calls.append(section["eviction_policy"])
            return True

    class Orch:
        draft, gamma = object(), 3
        engine = SpmdLeader(Eng(), broadcast=sent.append)

    cfg = load_config(None, {"memory.expert_cache.eviction_policy": "lfu"})
    apply_live_changes([("memory.expert_cache.eviction_policy", "impact_weighted_lru", "lfu"), ("speculation.mtp.max_depth", 3, 5)], Orch, cfg)
    assert calls == ["lfu"] and Orch.gamma == 5
    assert "configure_expert_cache" in MIRRORED and sent and sent[0][0] == "configure_expert_cache"      # announced to the other ranks
    apply_live_changes([("orchestrator.max_batch_size", 4, 8)], Orch, cfg)
    assert calls == ["lfu"]
