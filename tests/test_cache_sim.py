"""Offline expert-cache replay (CPU only, native cache bookkeeping)."""
import io
import json

from layerstorm_b200.utils import cache_sim


def test_trace_roundtrip(tmp_path):
    tr = cache_sim.synthetic_trace(5, 2, 16, 2, seed=3)
    p = str(tmp_path / "t.txt")
    cache_sim.write_trace(p, tr)
    assert cache_sim.read_trace(p) == tr
    assert len(tr) == 10 and all(len(set(ids)) == 2 for _, _, ids in tr)


def test_more_slots_and_prefetch_raise_the_hit_rate():
    tr = cache_sim.synthetic_trace(300, 3, 64, 4, zipf=1.2, stickiness=0.5, seed=1)
    small = cache_sim.simulate(tr, slots=8, policy="lru")
    big = cache_sim.simulate(tr, slots=32, policy="lru")
    assert small["hits"] + small["misses"] == 300 * 3 * 4 == big["hits"] + big["misses"]
    assert big["hit_rate"] > small["hit_rate"] + 0.1 and big["h2d_bytes"] < small["h2d_bytes"]
    assert cache_sim.simulate(tr, slots=64, policy="lru")["evictions"] == 0
    pf = cache_sim.simulate(tr, slots=16, policy="lru", prefetch_budget=4)
    base = cache_sim.simulate(tr, slots=16, policy="lru")
    assert pf["prefetched"] > 0 and pf["useful_prefetch"] > 0 and pf["misses"] < base["misses"]
    assert pf["demand_miss_bytes"] < base["demand_miss_bytes"]


def test_weighted_policy_and_decision_stream():
    tr = cache_sim.synthetic_trace(200, 2, 48, 4, zipf=1.3, stickiness=0.3, seed=2)
    out = io.StringIO()
    freq = cache_sim.simulate(tr, slots=12, weights=[0.1, 0.9, 0, 0, 0, 0, 0], decisions=out)
    lru = cache_sim.simulate(tr, slots=12, policy="lru")
    assert freq["hit_rate"] > lru["hit_rate"]                  # Zipf popularity: frequency beats pure recency
    lines = out.getvalue().splitlines()
    assert sum(l.startswith("M ") for l in lines) == freq["misses"] and sum(l.startswith("E ") for l in lines) == freq["evictions"]


def test_cli_prints_one_json_line(capsys):
    assert cache_sim.main(["--slots", "8", "--synthetic", "40,2,32,4", "--weights", "0.4,0.35,0.25,0,0,0,0"]) == 0
    rep = json.loads(capsys.readouterr().out.strip())
    assert rep["steps"] == 40 and rep["layers"] == 2 and 0 < rep["hit_rate"] < 1


def test_replay_projects_exposed_copy_time_and_the_cpu_offload_split():
    """With a copy rate the replay turns demand misses into exposed copy time per step; with a host expert time it also projects
    the split of every layer's misses between the copy engine and the host kernels (never worse than copying everything, never
    worse than the host alone, equal to the closed form for one layer)."""
    from layerstorm_b200.utils.cache_sim import simulate, synthetic_trace
    tr = synthetic_trace(40, 3, 48, 6, seed=5)
    base = simulate(tr, 12, slot_bytes=20 << 20)
    assert "projected" not in base
    r = simulate(tr, 12, slot_bytes=20 << 20, h2d_gbs=50.0)
    f = (20 << 20) / 50e6
    assert abs(r["projected"]["copy_ms_per_expert"] - f) < 1e-3
    assert abs(r["projected"]["exposed_copy_ms_per_step"] - r["misses"] * f / r["steps"]) < 1e-2
    fast = simulate(tr, 12, slot_bytes=20 << 20, h2d_gbs=50.0, cpu_expert_ms=0.05)["projected"]
    slow = simulate(tr, 12, slot_bytes=20 << 20, h2d_gbs=50.0, cpu_expert_ms=50.0)["projected"]
    assert fast["with_cpu_offload_ms_per_step"] < 0.3 * fast["exposed_copy_ms_per_step"]
    assert slow["with_cpu_offload_ms_per_step"] == slow["exposed_copy_ms_per_step"]          # a hopeless host takes nothing
    # one layer, one step, 5 misses, f = 0.4, c = 0.6: n = 2 on the host -> max(1.2, 1.2) = 1.2
    one = simulate([(0, 0, [1, 2, 3, 4, 5])], 8, slot_bytes=20000000, h2d_gbs=50.0, cpu_expert_ms=0.6)["projected"]
    assert abs(one["with_cpu_offload_ms_per_step"] - 1.2) < 1e-6
