"""CPU tests of the native (C++) runtime bookkeeping: page allocator and expert cache."""
import pytest

from layerstorm_b200 import build as _build

_build.build_all(only="runtime")

from layerstorm_b200.runtime import native as nt


def test_page_allocator_extend_fork_cow_rewind():
    pa = nt.PageAllocator([8, 4], page_tokens=16)
    pa.create(1)
    new = pa.extend(1, 40)
    assert new == [0, 1, 2] and pa.length(1) == 40 and pa.free_pages() == 5
    # truncating fork shares the pages that cover the prefix
    pa.fork(1, 2, 20)
    assert pa.pages(2) == [0, 1] and pa.refcount(0, 0) == 2 and pa.refcount(0, 1) == 2 and pa.refcount(0, 2) == 1
    # the child's frontier page (index 1, 4 tokens used) is shared: appending needs a private copy
    cow = pa.cow_frontier(2)
    assert cow is not None and cow[0] == 1
    assert pa.pages(2)[1] == cow[1] and pa.refcount(0, 1) == 1
    pa.extend(2, 33)
    assert len(pa.pages(2)) == 3
    # frozen holders never append
    pa.fork(1, 3, 32, frozen=True)
    with pytest.raises(nt.NativeError):
        pa.extend(3, 40)
    assert pa.cow_frontier(1) is None or True
    pa.rewind(1, 16)
    assert pa.pages(1) == [0]
    pa.destroy(2); pa.destroy(3); pa.destroy(1)
    assert pa.free_pages() == 8


def test_page_allocator_exhaustion_headroom_zones_promote():
    pa = nt.PageAllocator([4, 4], page_tokens=16)
    pa.create(1)
    pa.set_headroom(0, 1)
    pa.extend(1, 48)
    with pytest.raises(nt.KvPoolExhausted):
        pa.extend(1, 64)                       # last page is headroom
    pa.extend(1, 64, privileged=True)
    with pytest.raises(nt.KvPoolExhausted):
        pa.extend(1, 80, privileged=True)
    pa.rewind(1, 16)
    pa.set_headroom(0, 0)
    start = pa.claim_zone(0, 2)
    assert start >= 0 and pa.lent_pages(0) == 2 and pa.free_pages(0) == 1
    pa.release_zone(0, start, 2)
    assert pa.free_pages(0) == 3
    pa.create(7, pool=nt.POOL_SPECULATION)
    pa.extend(7, 20)
    pa.promote(7, nt.POOL_MAIN)
    assert pa.free_pages(1) == 4 and pa.free_pages(0) == 1
    assert nt.dcp_rank_for_token(130, 64, 4) == 2 and nt.dcp_local_index(130, 64, 4) == 2
    assert nt.dcp_rank_for_token(64 * 5 + 3, 64, 4) == 1 and nt.dcp_local_index(64 * 5 + 3, 64, 4) == 64 + 3


def test_expert_cache_two_phase_lock_evict():
    ec = nt.ExpertCache(3, 1, "lru")
    events = []
    ec.set_listener(lambda l, e, s, r: events.append((l, e, r)))
    s0 = ec.reserve(0, 5)
    assert not ec.is_ready(0, 5)
    ec.mark_ready(0, 5)
    assert ec.is_ready(0, 5) and events == [(0, 5, True)]
    ec.reserve(0, 6); ec.mark_ready(0, 6)
    ec.reserve(1, 5); ec.mark_ready(1, 5)
    with pytest.raises(nt.NativeError):
        ec.reserve(2, 1)                                    # stable zone full, no fallback
    s = ec.reserve(2, 1, fallback=True)                     # spills into the streaming zone
    assert ec.slot_info(s)["zone"] == nt.ZONE_STREAMING
    ec.cancel(2, 1)                                         # failed fill: slot is free again
    assert ec.lookup(2, 1) == -1
    ec.lock(0, 5)
    with pytest.raises(nt.NativeError):
        ec.evict(0, 5)
    ec.touch(0, 6); ec.touch(0, 5)
    v = ec.pick_victim()
    assert v is not None and (v[1], v[2]) == (1, 5)         # least recently used, unlocked
    ec.unlock(0, 5)
    ec.evict(1, 5)
    assert events[-1] == (1, 5, False)
    gen = ec.add_elastic_zone(2)
    assert ec.n_slots() == 6
    ec.reserve(3, 3); ec.reserve(3, 4)
    s = ec.reserve(3, 5)
    with pytest.raises(nt.NativeError):
        ec.remove_elastic_zone(gen)
    for e in (3, 4, 5):
        ec.cancel(3, e)
    ec.remove_elastic_zone(gen)
    assert ec.n_slots() == 4 and ec.lookup(0, 5) == s0


def test_stats():
    es = nt.ExpertStats(8, alpha=0.5)
    for _ in range(6):
        es.observe([1, 3], [0.7, 0.3])
    es.observe([2], [1.0])
    assert es.frequency(1) > 0.4 and es.frequency(5) == 0 and abs(es.weight(1) - 0.7) < 0.05
    assert es.recency(2) == 1.0 and 0 < es.recency(1) < 1 and es.autocorr(1) > 0.4 and len(es.frequencies()) == 8
    cg = nt.CoactivationGraph(8, 0.99)
    for _ in range(10):
        cg.observe([0, 1]); cg.observe([2, 3]); cg.observe([4, 5, 6, 7])
    part = cg.partition(4)
    assert part[0] == part[1] and part[2] == part[3] and sorted(part.count(g) for g in range(4)) == [2, 2, 2, 2]
    wd = nt.WorkloadDetector(4, z=3.0)
    base = [0.5, 0.5, 0.0, 0.0]
    assert not any(wd.observe([b + 0.01 * (i % 3) for b in base]) for i in range(12))
    assert wd.observe([0.0, 0.0, 0.5, 0.5]) and wd.shifts() == 1
    at = nt.AcceptanceTracker(0.5, 4)
    at.record(1, 8, 6); at.record(1, 8, 2); at.record(2, 4, 4)
    assert abs(at.global_rate() - 0.6) < 1e-6 and abs(at.request_rate(1) - 0.5) < 1e-6 and at.request_rate(2) == 1.0
    assert 1.0 < at.expected_tokens(4) < 5.0
    at.forget(1)
    assert at.request_rate(1) == 0.0


def test_ring_snapshot_trace(tmp_path):
    import threading
    r = nt.SpscRing(8, 32)
    with pytest.raises(ValueError):
        nt.SpscRing(6, 32)
    assert r.pop() is None
    for i in range(8):
        assert r.push(bytes([i]) * 4)
    assert not r.push(b"x") and len(r) == 8              # full -> back-pressure
    assert r.pop()[:4] == b"\x00" * 4 and r.push(b"zz") and len(r) == 8
    got = []
    ring = nt.SpscRing(64, 16)
    def consumer():
        while len(got) < 2000:
            m = ring.pop()
            if m is not None:
                got.append(int.from_bytes(m[:4], "little"))
    th = threading.Thread(target=consumer); th.start()
    i = 0
    while i < 2000:
        if ring.push(i.to_bytes(4, "little")):
            i += 1
    th.join()
    assert got == list(range(2000))
    s = nt.StateSnapshot(64)
    s.begin(); s.write(0, b"abcd"); s.begin(); s.write(4, b"efgh")
    assert s.read(0, 8)[0] is None                        # writer active: no consistent copy
    s.end(); assert s.read(0, 8)[0] is None               # nested transaction still open
    s.end()
    data, ver = s.read(0, 8)
    assert data == b"abcdefgh" and ver > 0
    t = nt.PerfTrace(16)
    for tok in range(5):
        t.record(1, token=tok); t.record(2, token=tok)
    tot, n = t.span_ns(1, 2)
    assert n == 5 and tot >= 0 and t.count() == 10
    for _ in range(10):
        t.record(3)
    assert t.count() == 16 and t.dropped() == 4
    t.dump_csv(str(tmp_path / "t.csv"))
    assert len(open(tmp_path / "t.csv").read().splitlines()) == 17


def test_loader_solver_tiers_agree_with_brute_force():
    import itertools, random
    M = 3
    sv = nt.LoaderSolver(a_ns=[16000] * M, b_ns=[64000] * M, rate_bpus=[[50000] * M, [30000] * M], lat_ns=[[9000] * M, [12000] * M],
                         egress_bpus=[80000, 60000], batch_p=64, recon_ns=20000, evict_ns=30000)
    rng = random.Random(0)
    for trial in range(8):
        n = rng.randint(3, 6)
        bank = [rng.randint(0, 1) for _ in range(n)]
        nbytes = [rng.choice([14_000_000, 25_000_000]) for _ in range(n)]
        resident = [[rng.random() < 0.3 for _ in range(M)] for _ in range(n)]
        free = [rng.randint(0, 3) for _ in range(M)]
        assign, cost, tier = sv.solve(bank, nbytes, resident, free, tier=0)
        assert tier == 1
        brute = min(sv.evaluate(bank, nbytes, resident, free, list(a)) for a in itertools.product(range(M), repeat=n))
        assert cost == brute == sv.evaluate(bank, nbytes, resident, free, assign)
        for t in (2, 3):
            a2, c2, used = sv.solve(bank, nbytes, resident, free, tier=t)
            assert used == t and c2 >= brute and c2 == sv.evaluate(bank, nbytes, resident, free, a2)
            assert c2 <= 2 * brute
    # a resident expert stays where it is when that is free of charge
    a, c, _ = sv.solve([0], [14_000_000], [[False, True, False]], [1, 1, 1])
    assert a == [1] and c == 16000 + 64000


def test_page_swap_out_and_in_for_kv_tiering():
    """Tiering of an active sequence: a completely filled private page behind the frontier gives its HBM page back (block-table
    entry -1) and gets a fresh one on promotion; shared pages, the frontier page and holes cannot be swapped or forked."""
    from layerstorm_b200.runtime import native as rt
    pa = rt.PageAllocator([6], 16)
    pa.create(0)
    pa.extend(0, 40)                                   # pages 0, 1 full, page 2 holds 8 tokens
    assert pa.free_pages() == 3
    released = pa.swap_out(0, 0)
    assert pa.pages(0)[0] == -1 and pa.free_pages() == 4 and released >= 0
    with pytest.raises(rt.NativeError):
        pa.swap_out(0, 0)                              # already out
    with pytest.raises(rt.NativeError):
        pa.swap_out(0, 2)                              # the frontier page is not full
    with pytest.raises(rt.NativeError):
        pa.fork(0, 1, 32)                              # a hole cannot be shared
    pa.extend(0, 64)                                   # growing past a hole works
    assert len(pa.pages(0)) == 4 and pa.pages(0)[0] == -1
    pg = pa.swap_in(0, 0)
    assert pa.pages(0)[0] == pg >= 0
    pa.fork(0, 1, 32)
    with pytest.raises(rt.NativeError):
        pa.swap_out(0, 1)                              # shared with the fork
    pa.destroy(1)
    pa.swap_out(0, 1)
    pa.rewind(0, 8)                                    # releasing a range that contains a hole
    pa.destroy(0)
    assert pa.free_pages() == 6
