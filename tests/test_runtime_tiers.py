"""Host runtime, second batch: transfer engine, host arena / NUMA sizing, NVMe tier, expert lifecycle,
zone rebalancer, KV tier table, VRAM planner, determinism registry, buffer registry (all CPU)."""
import os
import time

import pytest

from layerstorm_b200 import build as _build

_build.build_all(verbose=False, only="runtime")

from layerstorm_b200.runtime import native as rt


# ---------------------------------------------------------------- transfer engine
def test_transfer_dedup_priority_waterline_and_cancel():
    te = rt.TransferEngine(n_gpus=2, levels=3, waterline=2)
    a = te.submit(3, 7, gpu=0, priority=2, nbytes=1 << 20)
    b = te.submit(3, 8, gpu=0, priority=1, nbytes=1 << 20)
    c = te.submit(3, 9, gpu=0, priority=2, nbytes=1 << 20)
    assert 0 < a < b < c
    assert te.submit(3, 7, gpu=0, priority=0, nbytes=1 << 20) == a and te.dedup_hits() == 1     # same key: same token, priority raised
    assert te.info(a)["priority"] == 0 and te.find(3, 7) == a
    assert te.submit(3, 7, gpu=1, priority=2) != a                                             # other GPU = other transfer
    assert te.queued(0) == 3
    first, second = te.next_to_issue(0, 1000), te.next_to_issue(0, 1000)
    assert (first, second) == (a, b)                                                           # priority order, FIFO inside a level
    assert te.next_to_issue(0, 1000) == 0 and te.in_flight(0) == 2                             # waterline reached
    assert te.cancel(c) == 1                                                                   # queued: dropped now
    assert te.cancel(b) == 2                                                                   # in flight: deferred
    te.complete(a, 1000 + 1_000_000)                                                           # 1 MiB in 1 ms ~ 1.05 GB/s
    te.complete(b, 1000 + 2_000_000)
    done = te.poll()
    assert [(t, s) for t, s, *_ in done] == [(c, 3), (a, 2), (b, 3)]
    assert abs(te.bandwidth_gbs(0, 0) - (0.8 * 1.048576 + 0.2 * 0.524288)) < 1e-6
    assert te.find(3, 7) == 0 and te.in_flight(0) == 0
    d = te.submit(3, 7, gpu=0, priority=1)
    assert d > c                                                                               # tokens never repeat
    with pytest.raises(rt.NativeError):
        te.complete(d)                                                                         # not in flight


# ---------------------------------------------------------------- arena / NUMA
def test_numa_topology_and_budget(tmp_path):
    for node, (tot, free, cpus) in {0: (64 << 20, 32 << 20, "0-3,8"), 1: (128 << 20, 100 << 20, "")}.items():
        d = tmp_path / f"node{node}"
        d.mkdir()
        (d / "meminfo").write_text(f"Node {node} MemTotal:       {tot // 1024} kB\nNode {node} MemFree:        {free // 1024} kB\n")
        (d / "cpulist").write_text(cpus + "\n")
    topo = rt.numa_topology(str(tmp_path))
    assert [n["id"] for n in topo] == [0, 1]
    assert topo[0]["total_bytes"] == 64 << 20 and topo[0]["n_cpus"] == 5
    assert topo[1]["n_cpus"] == 0 and topo[1]["free_bytes"] == 100 << 20             # memory-only node
    assert rt.host_pool_budget("fraction_total", 0.5, 128 << 20, 100 << 20) == 64 << 20
    assert rt.host_pool_budget("fraction_free", 0.9, 128 << 20, 100 << 20) == int(0.9 * (100 << 20))
    assert rt.host_pool_budget("fraction_total", 0.9, 128 << 20, 100 << 20, reserve_bytes=10 << 20) == 90 << 20   # capped by what is free
    assert rt.host_pool_budget("absolute_gb", 1.0, 1 << 40, 1 << 39) == 1 << 30
    assert isinstance(rt.numa_topology(), list)


def test_host_arena_lru_refs_states_and_meta(tmp_path):
    ar = rt.HostArena(4096, 3, numa_node=0, memfd=True, thp=False)
    assert ar.nbytes == 3 * 4096 and ar.fd >= 0
    t = ar.tensor()
    slots = {}
    for e in range(3):
        s, ev = ar.begin_load(0, e)
        assert ev is None and ar.lookup(0, e) == -1              # not visible while loading
        t[s].fill_(e + 1)
        ar.finish_load(s)
        slots[e] = s
    assert ar.lookup(0, 1) == slots[1]                          # touch 1 -> LRU order is 0, 2, 1
    ar.ref(slots[0], +1)                                        # 0 is being copied to a GPU: not evictable
    s, ev = ar.begin_load(0, 3)
    assert ev == (0, 2) and s == slots[2]
    with pytest.raises(rt.NativeError):
        ar.begin_load(0, 3)                                     # already loading
    ar.finish_load(s, ok=False)                                 # failed load leaves an empty slot, not a stale expert
    assert ar.lookup(0, 3) == -1 and ar.slot_info(s)["state"] == rt.HostArena.EMPTY
    assert int(t[slots[0]][0]) == 1
    ar.save_meta(tmp_path / "meta", tag=42)
    ar2 = rt.HostArena(4096, 3, memfd=False)
    assert ar2.load_meta(tmp_path / "meta", tag=41) == rt.ERR_FORMAT        # other model: start empty
    assert ar2.load_meta(tmp_path / "meta", tag=42) == 2 and ar2.lookup(0, 1) == slots[1]
    with pytest.raises(rt.NativeError):
        ar.wipe()                                               # a slot is referenced
    ar.ref(slots[0], -1)
    ar.wipe()
    assert ar.stats()["active"] == 0 and ar.stats()["evictions"] == 1


# ---------------------------------------------------------------- NVMe tier
def test_nvme_tier_roundtrip_async_and_capacity(tmp_path):
    drives = [tmp_path / "d0", tmp_path / "d1"]
    for d in drives:
        d.mkdir()
    nv = rt.NvmeTier(drives, capacity_bytes=3 * 8192, queue_depth=2, workers=2)
    blobs = {e: bytes([e]) * 8192 for e in range(3)}
    for e, b in blobs.items():
        nv.write(5, e, b)
    assert (drives[0] / "L5" / "E0.bin").exists() and (drives[1] / "L5" / "E1.bin").exists() and (drives[0] / "L5" / "E2.bin").exists()
    assert nv.used() == 3 * 8192 and nv.size_of(5, 1) == 8192 and nv.size_of(5, 9) == -1
    with pytest.raises(rt.NativeError):
        nv.write(5, 3, b"x" * 8192)                              # over capacity
    nv.write(5, 1, b"\x07" * 8192)                               # rewrite in place does not grow usage
    assert nv.used() == 3 * 8192 and nv.read(5, 1, 8192) == b"\x07" * 8192
    ar = rt.HostArena(8192, 2)
    t1 = nv.read_async(5, 0, ar.base, 8192)
    t2 = nv.read_async(5, 2, ar.base + 8192, 8192)
    assert t1 and t2
    done = {}
    for _ in range(200):
        done.update(dict(nv.poll()))
        if len(done) == 2:
            break
        time.sleep(0.01)
    assert done == {t1: 0, t2: 0}
    assert bytes(ar.tensor()[0][:4].tolist()) == b"\x00" * 4 and int(ar.tensor()[1][0]) == 2
    t3 = nv.read_async(5, 8, ar.base, 8192)                      # missing file -> error status, not an exception
    for _ in range(200):
        r = nv.poll()
        if r:
            assert r == [(t3, rt.ERR_NOT_FOUND)]
            break
        time.sleep(0.01)
    nv.evict(5, 0)
    assert nv.used() == 2 * 8192 and not (drives[0] / "L5" / "E0.bin").exists()


# ---------------------------------------------------------------- lifecycle
def test_expert_lifecycle_walks_cold_to_hot_and_protects_interest():
    L = rt.ExpertLifecycle
    m = L()
    act, tok = m.ensure_resident(2, 11, gpu=0)
    assert act == L.ACT_READ_NVME and tok > 0
    m.begin_host_load(2, 11)
    assert m.ensure_resident(2, 11, gpu=1)[0] == L.ACT_WAIT            # another GPU sees the load in progress
    assert m.on_event(2, 11, 0, L.EV_NVME_DONE) == L.ACT_RESERVE_SLOT
    assert m.get(2, 11, 1)[0] == L.WARM                                # host tier is shared between GPUs
    assert m.on_event(2, 11, 0, L.EV_SLOT_DENIED) == L.ACT_RESERVE_SLOT  # caller must make room: reserve never evicts
    assert m.on_event(2, 11, 0, L.EV_SLOT_RESERVED) == L.ACT_START_H2D
    assert m.on_event(2, 11, 0, L.EV_H2D_STARTED) == L.ACT_WAIT
    with pytest.raises(rt.NativeError):
        m.on_event(2, 11, 0, L.EV_HOST_EVICTED)                        # the copy still reads the host slot
    assert m.on_event(2, 11, 0, L.EV_H2D_DONE) == L.ACT_NONE
    assert m.get(2, 11, 0) == (L.WARM, L.HOT, 1) and m.loads() == 1
    assert m.ensure_resident(2, 11, 0) == (L.ACT_NONE, tok)            # same token while resident
    with pytest.raises(rt.NativeError) as e:
        m.on_event(2, 11, 0, L.EV_EVICT_REQUESTED)
    assert e.value.code == rt.ERR_BUSY                                 # interest 2: about to run
    m.release(2, 11, 0); m.release(2, 11, 0)
    assert m.on_event(2, 11, 0, L.EV_EVICT_REQUESTED) == L.ACT_WAIT
    with pytest.raises(rt.NativeError):
        m.on_event(2, 11, 0, L.EV_H2D_DONE)                            # event does not fit the state
    m.on_event(2, 11, 0, L.EV_DRAINED)
    assert m.get(2, 11, 0)[1] == L.ABSENT and m.evictions() == 1
    assert m.ensure_resident(2, 11, 0)[0] == L.ACT_RESERVE_SLOT        # still warm in host memory


# ---------------------------------------------------------------- zone rebalancer
def test_zone_rebalancer_hysteresis_and_quiesce():
    Z = rt.ZoneRebalancer
    z = Z(total_kv_pages=1000, pages_per_zone=200, low_water=0.5, high_water=0.85, max_zones=2)
    assert z.step(kv_used=100, miss_rate=0.0) == (Z.NONE, -1)          # no expert pressure: nothing to do
    a, g1 = z.step(kv_used=100, miss_rate=0.2)
    assert a == Z.LEND and g1 == 1
    z.on_lent(g1)
    a, g2 = z.step(kv_used=100, miss_rate=0.2)
    assert a == Z.LEND and g2 == 2
    z.on_lent(g2)
    assert z.lent_pages() == 400 and z.step(100, 0.2)[0] == Z.NONE      # max zones
    assert z.step(kv_used=450, miss_rate=0.2)[0] == Z.NONE              # 450/600 = 0.75: between the marks
    a, g = z.step(kv_used=540, miss_rate=0.2)                           # 0.9 > high water: newest zone goes back
    assert (a, g) == (Z.BEGIN_RECLAIM, g2)
    with pytest.raises(rt.NativeError):
        z.on_reclaimed(g1)                                              # not quiescing
    assert z.step(540, 0.2, zone_occupancy=3) == (Z.NONE, g2)           # wait for the drain
    assert z.step(540, 0.2, zone_occupancy=0) == (Z.FINISH_RECLAIM, g2)
    z.on_reclaimed(g2)
    assert z.n_zones() == 1 and z.lent_pages() == 200
    assert z.step(540, 0.2)[0] == Z.NONE                                # 540/800 = 0.675: no flapping


# ---------------------------------------------------------------- KV tier table
def test_kv_tier_table_demote_fork_rewind_and_row_cache():
    T = rt.KvTierTable
    kt = T(page_tokens=16, hot_window_tokens=64, cold_slots=4, row_cache_rows=2)
    kt.create(1)
    assert kt.demotion_candidates(1, 70) == []                          # (70-64)/16 = 0 whole pages behind the window
    assert kt.demotion_candidates(1, 130) == [0, 1, 2, 3]
    s0, s1 = kt.demote(1, 0), kt.demote(1, 1)
    assert s0 != s1 and kt.demote(1, 0) == s0 and kt.free_cold_slots() == 2
    assert kt.demotion_candidates(1, 130) == [2, 3]
    kt.fork(1, 2, prefix_pages=2)                                       # child shares both cold pages
    assert kt.where(2, 0) == s0
    kind, ref, cold = kt.classify(1, layer=3, rows=[5, 40, 100, 20])
    assert kind == [T.COLD, T.HOT_PAGE, T.HOT_PAGE, T.COLD] and ref[0] == s0 and ref[3] == s1 and cold == 2
    l0, l1 = kt.cache_row(1, 3, 5), kt.cache_row(1, 3, 20)
    kind, ref, cold = kt.classify(1, 3, [5, 20])
    assert kind == [T.ROW_CACHE, T.ROW_CACHE] and ref == [l0, l1] and cold == 0
    assert kt.cache_row(1, 3, 7) == l0                                  # LRU line reused (row 5 was least recently used)
    assert kt.classify(1, 3, [5])[0] == [T.COLD]
    kt.truncate(1, 10)                                                  # rewind into page 0: the parent drops page 1
    assert kt.free_cold_slots() == 2                                    # the child still holds both slots
    assert kt.promote(2, 1) == s1 and kt.free_cold_slots() == 3
    kt.destroy(2)
    assert kt.free_cold_slots() == 3 and kt.where(1, 0) == s0           # page 0 is still the parent's
    kt.destroy(1)
    assert kt.free_cold_slots() == 4
    st = kt.stats()
    assert st["demotions"] >= 2 and st["promotions"] == 1 and st["row_hits"] == 2


# ---------------------------------------------------------------- planner / determinism / buffers
def test_vram_plan_regions_and_failure():
    G = 1 << 30
    p = rt.vram_plan(total_bytes=180 * G, weights_bytes=10 * G, workspace_bytes=G, kv_bytes_per_page=64 * 528 * 11, kv_pages=20000,
                     spec_pool_fraction=0.1, recurrent_bytes_per_seq=140 << 20, recurrent_seqs=8, expert_slot_bytes=12 << 20,
                     expert_slots_wanted=289 * 42, stable_zone_fraction=0.7, safety_bytes=G)
    r = p["regions"]
    order = list(rt.VRAM_REGIONS)
    for a, b in zip(order[:-1], order[1:]):
        assert r[a]["offset"] + r[a]["size"] <= r[b]["offset"] + (1 if r[b]["size"] == 0 else 0) or r[b]["size"] == 0
    assert all(v["offset"] % (2 << 20) == 0 for k, v in r.items() if k != "expert_stable")
    assert p["kv_spec_pages"] == 2000 and p["expert_stable_slots"] == 289 * 42 and p["expert_streaming_slots"] == 0   # everything fits
    q = rt.vram_plan(total_bytes=80 * G, weights_bytes=10 * G, workspace_bytes=G, kv_bytes_per_page=1 << 20, kv_pages=4096,
                     expert_slot_bytes=14 << 20, expert_slots_wanted=289 * 42, stable_zone_fraction=0.7)
    tot = q["expert_stable_slots"] + q["expert_streaming_slots"]
    assert 0 < tot < 289 * 42 and abs(q["expert_stable_slots"] / tot - 0.7) < 0.01
    assert r["safety"]["size"] >= G
    with pytest.raises(rt.NativeError) as e:
        rt.vram_plan(total_bytes=16 * G, weights_bytes=10 * G, workspace_bytes=G, kv_bytes_per_page=1 << 20, kv_pages=8192)
    assert "kv_main" in str(e.value)


def test_determinism_registry_refuses_contrary_pins():
    d = rt.Determinism()
    assert "deterministic_reduce" in d.knobs() and d.get("spec_round_governor") == 1
    d.set_flags(deterministic=True)
    assert d.get("atomic_accumulate") == 0 and d.get("spec_round_governor") == 1       # free under run-to-run determinism
    d.set_flags(identity=True)
    assert d.get("spec_round_governor") == 0 and d.get("ep_combine_fp32") == 1
    with pytest.raises(rt.NativeError):
        d.pin("spec_round_governor", 1)                                                # contradicts the active super-flag
    d2 = rt.Determinism()
    d2.pin("atomic_accumulate", 1)
    with pytest.raises(rt.NativeError) as e:
        d2.set_flags(deterministic=True)
    assert "atomic_accumulate" in str(e.value)
    with pytest.raises(rt.NativeError):
        d2.pin("no_such_knob", 1)


def test_buffer_registry():
    b = rt.BufferRegistry()
    i = b.add("kv_main", 0x1000, 4096, gpu=1)
    j = b.add("logits", 0x9000, 256)
    assert (i, j) == (0, 1) and b.find("logits") == 1 and len(b) == 2
    assert b.get(i) == (0x1000, 4096, 1)
    assert b.contains(i, 0x1800, 2048) and not b.contains(i, 0x1800, 4096) and not b.contains(7, 0, 1)
    with pytest.raises(rt.NativeError):
        b.add("logits", 0, 1)
    with pytest.raises(rt.NativeError):
        b.find("nope")


# ---------------------------------------------------------------- CPU expert kernels
@pytest.mark.parametrize("fmt,H,F", [("bf16", 64, 48), ("fp8_e4m3", 256, 128), ("nvfp4", 256, 128), ("gguf_q4_k", 256, 256)])
def test_cpu_expert_ffn_reads_gpu_slot_images(fmt, H, F):
    import ctypes
    import torch
    from layerstorm_b200.models.device_model import ExpertArena, QLinear, expert_layout
    cpu = rt.CpuExperts(3)
    assert cpu.threads == 3
    g = torch.Generator().manual_seed(0)
    E, S, T = 4, 2, 7
    ef = expert_layout(fmt, H, F)
    ar = ExpertArena(ef, E, E, "cpu")
    deq = {}
    for e in range(E):
        mats = [torch.randn(F, H, generator=g) * 0.05, torch.randn(F, H, generator=g) * 0.05, torch.randn(H, F, generator=g) * 0.05]
        ar.write_expert(e, *(QLinear.from_float(m, fmt, "cpu") for m in mats))
        deq[e] = [m.double() for m in ar.read_expert(e, fmt)]
    x = torch.randn(T, H, generator=g)

    def ref_ffn(e, xv, limit):
        gate, up, down = deq[e]
        gv, uv = torch.clamp(xv.double() @ gate.T, max=limit), torch.clamp(xv.double() @ up.T, -limit, limit)
        return (torch.nn.functional.silu(gv) * uv) @ down.T

    y = cpu.ffn(ctypes.addressof(ef), ar.data[1], x, limit=3.0)
    want = ref_ffn(1, x, 3.0)
    assert float((y.double() - want).abs().max() / want.abs().max()) < 1e-5
    ids = torch.randint(0, E, (T, S), generator=g).int()
    ids[2, 1] = 3
    wts = torch.rand(T, S, generator=g)
    slots = {e: ar.data[e] for e in range(E) if e != 3}            # expert 3 is not available on the host
    out = cpu.moe_layer(ctypes.addressof(ef), slots, E, x, ids, wts, limit=3.0)
    want = torch.zeros(T, H, dtype=torch.float64)
    for t in range(T):
        for s in range(S):
            if int(ids[t, s]) != 3:
                want[t] += float(wts[t, s]) * ref_ffn(int(ids[t, s]), x[t:t + 1], 3.0)[0]
    assert float((out.double() - want).abs().max() / want.abs().max()) < 1e-5


def test_calibration_fit_document_and_solver(tmp_path):
    import json
    from layerstorm_b200.runtime import calibration as cal
    counts = [1, 2, 4, 8, 16, 64, 65, 128]
    a, b, P = 9000.0, 30000.0, 64
    times = [a * c + b * -(-c // P) for c in counts]
    fa, fb = cal.fit_compute_curve(counts, times, P)
    assert abs(fa - a) / a < 1e-6 and abs(fb - b) / b < 1e-6
    doc = {"version": 2, "batch_p": P, "devices": [{"a_ns": fa, "b_ns": fb}, {"a_ns": 2 * fa, "b_ns": fb}],
           "banks": [{"rate_bytes_per_us": [50000, 25000], "latency_ns": [8000, 9000], "egress_bytes_per_us": 60000}],
           "recon_ns": 12000, "evict_ns": 4000}
    p = tmp_path / "cal.json"
    p.write_text(json.dumps(doc))
    assert cal.calibrate(mode="loaded", path=str(p))["devices"][1]["a_ns"] == 2 * fa
    (tmp_path / "old.json").write_text(json.dumps({"version": 1}))
    with pytest.raises(ValueError):
        cal.calibrate(mode="loaded", path=str(tmp_path / "old.json"))
    solver = cal.solver_from_calibration(doc)
    assign, cost, tier = solver.solve([0] * 6, [14 << 20] * 6, [[1, 0]] * 3 + [[0, 0]] * 3, [4, 4])
    assert len(assign) == 6 and cost > 0 and tier == 1
    assert all(x == 0 for x in assign[:3])                 # resident experts stay on the device that holds them


def test_arena_holder_keeps_slab_across_clients(tmp_path):
    import subprocess, sys, time as _t
    import torch
    from layerstorm_b200.runtime.arena_holder import HolderClient
    sock = str(tmp_path / "holder.sock")
    proc = subprocess.Popen([sys.executable, "-m", "layerstorm_b200.runtime.arena_holder", "serve", "--socket", sock],
                            cwd=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    try:
        c = HolderClient(sock)
        for _ in range(100):
            if c.alive():
                break
            _t.sleep(0.05)
        assert c.alive()
        ar = rt.HostArena(4096, 4, memfd=True, thp=False)
        s, _ = ar.begin_load(3, 9)
        ar.tensor()[s].fill_(0x5A)
        ar.finish_load(s)
        ar.save_meta(tmp_path / "meta", tag=7)
        c.put("gpu0", ar, tag=7)
        del ar                                                  # the engine process goes away; the holder keeps the slab
        got = HolderClient(sock).get("gpu0")
        assert got is not None
        ar2, tag = got
        assert tag == 7 and ar2.load_meta(tmp_path / "meta", tag=7) == 1
        s2 = ar2.lookup(3, 9)
        assert s2 == s and int(ar2.tensor()[s2][100]) == 0x5A   # contents survived
        st = c.status()
        assert st["arenas"]["gpu0"]["n_slots"] == 4
        with pytest.raises(ValueError):
            c.wipe("gpu0", " ")
        assert c.wipe("gpu0", "test teardown") and HolderClient(sock).get("gpu0") is None
        assert c.status()["wipes"][-1]["reason"] == "test teardown"
    finally:
        HolderClient(sock).shutdown()
        proc.wait(timeout=10)
