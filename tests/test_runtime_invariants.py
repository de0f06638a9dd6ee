"""Randomised operation sequences against the native page allocator and expert cache: conservation and reference-count invariants."""
import random

import pytest

from layerstorm_b200 import build as _build

_build.build_all(only="runtime")

from layerstorm_b200.runtime import native as rt

PAGE = 4


def _check_pages(pa, live, total):
    """Every page's refcount equals the number of live sequences holding it; free + held = total."""
    held = {}
    for s in live:
        pages = pa.pages(s)
        assert len(pages) == -(-pa.length(s) // PAGE), (s, pa.length(s), pages)
        assert len(set(pages)) == len(pages)
        for p in pages:
            held[p] = held.get(p, 0) + 1
    for p, n in held.items():
        assert pa.refcount(0, p) == n, (p, n, pa.refcount(0, p))
    assert pa.free_pages(0) + len(held) == total


@pytest.mark.parametrize("seed", range(6))
def test_page_allocator_random_walk(seed):
    rng = random.Random(seed)
    total = 40
    pa = rt.PageAllocator([total], PAGE)
    live, next_id = [], 0
    for _ in range(400):
        op = rng.choice(["create", "extend", "extend", "fork", "rewind", "destroy"])
        try:
            if op == "create" and len(live) < 8:
                pa.create(next_id)
                live.append(next_id)
                next_id += 1
            elif op == "extend" and live:
                s = rng.choice(live)
                cow = pa.cow_frontier(s)                          # a shared frontier page becomes private before it is written
                if cow is not None:
                    assert pa.refcount(0, cow[1]) == 1
                pa.extend(s, pa.length(s) + rng.randint(1, 9))
            elif op == "fork" and live and len(live) < 8:
                parent = rng.choice(live)
                pa.fork(parent, next_id, rng.randint(0, pa.length(parent)))
                live.append(next_id)
                next_id += 1
            elif op == "rewind" and live:
                s = rng.choice(live)
                pa.rewind(s, rng.randint(0, pa.length(s)))
            elif op == "destroy" and live:
                s = live.pop(rng.randrange(len(live)))
                pa.destroy(s)
        except rt.KvPoolExhausted:
            pass                                                  # a full pool refuses; state must stay consistent
        _check_pages(pa, live, total)
    for s in live:
        pa.destroy(s)
    assert pa.free_pages(0) == total


@pytest.mark.parametrize("seed", range(4))
def test_expert_cache_random_walk(seed):
    rng = random.Random(100 + seed)
    n_slots = 6
    ec = rt.ExpertCache(4, 2, ["impact_weighted_lru", "lru", "lfu"][seed % 3])
    if seed == 3:
        ec.set_weights("impact_weighted_lru", [0.4, 0.35, 0.25, 0.1, 0.1, 0.1, 0.1])
    state = {}                                                    # (layer, expert) -> "reserved" | "ready"; locks counted separately
    locks = {}
    for _ in range(600):
        key = (rng.randint(0, 1), rng.randint(0, 9))
        op = rng.choice(["reserve", "ready", "lock", "unlock", "evict", "victim", "touch", "cancel", "step"])
        if op == "reserve" and key not in state:
            try:
                ec.reserve(*key, zone=rng.randint(0, 1), fallback=True)
                state[key] = "reserved"
            except rt.NativeError:
                assert len(state) == n_slots                      # refused only when every slot is taken
        elif op == "ready" and state.get(key) == "reserved":
            ec.mark_ready(*key)
            state[key] = "ready"
        elif op == "cancel" and state.get(key) == "reserved":
            ec.cancel(*key)
            del state[key]
        elif op == "lock" and state.get(key) == "ready":
            ec.lock(*key)
            locks[key] = locks.get(key, 0) + 1
        elif op == "unlock" and locks.get(key, 0) > 0:
            ec.unlock(*key)
            locks[key] -= 1
        elif op == "touch" and key in state:
            ec.touch(*key, rng.random())
        elif op == "step":
            ec.end_step()
        elif op == "evict" and key in state:
            try:
                ec.evict(*key)
                assert state[key] == "ready" and locks.get(key, 0) == 0
                del state[key]
            except rt.NativeError:
                assert state[key] == "reserved" or locks.get(key, 0) > 0      # busy entries cannot be evicted
        elif op == "victim":
            v = ec.pick_victim(-1)
            evictable = [k for k, st in state.items() if st == "ready" and locks.get(k, 0) == 0]
            if v is None:
                assert not evictable
            else:
                assert (v[1], v[2]) in evictable
        # residency agrees with the model
        for k, st in state.items():
            assert ec.lookup(*k) >= 0 and ec.is_ready(*k) == (st == "ready")
        assert ec.count(-1, rt.SLOT_READY) == sum(1 for st in state.values() if st == "ready")


@pytest.mark.parametrize("seed", range(4))
def test_transfer_engine_random_walk(seed):
    """Submissions de-duplicate on (layer, expert, gpu, direction); at most ``waterline`` transfers are in flight per GPU; every
    transfer is reported by poll exactly once, as done or cancelled; the queue drains."""
    rng = random.Random(200 + seed)
    W = 3
    te = rt.TransferEngine(n_gpus=2, levels=3, waterline=W)
    live = {}                                                    # token -> key of transfers not yet reported
    active = set()                                               # tokens still queued or in flight (what a new request can ride on)
    flying = {0: set(), 1: set()}
    reported = {}
    now = 0

    def drain_poll():
        for tok, state, layer, expert, gpu in te.poll(64):
            assert tok not in reported and state in (2, 3), (tok, state)
            reported[tok] = state
            assert live.pop(tok) == (layer, expert, gpu)
            flying[gpu].discard(tok)

    for _ in range(800):
        now += 1000
        op = rng.choice(["submit", "submit", "issue", "issue", "complete", "cancel", "poll"])
        if op == "submit":
            key = (rng.randint(0, 2), rng.randint(0, 7), rng.randint(0, 1))
            before = te.dedup_hits()
            tok = te.submit(key[0], key[1], key[2], 0, rng.randint(0, 2), 1 << 20)
            assert tok != 0
            dup = [t for t, k in live.items() if k == key and t in active]
            if dup:
                assert tok == dup[0] and te.dedup_hits() == before + 1      # the same expert to the same GPU rides on the first request
            else:
                live[tok] = key
                active.add(tok)
            assert te.find(key[0], key[1], key[2], 0) == tok
        elif op == "issue":
            g = rng.randint(0, 1)
            tok = te.next_to_issue(g, now)
            if tok:
                assert tok in live and live[tok][2] == g and te.info(tok)["state"] == 1
                flying[g].add(tok)
            else:
                assert te.in_flight(g) >= W or te.queued(g) == 0
        elif op == "complete":
            g = rng.randint(0, 1)
            if flying[g]:
                tok = rng.choice(sorted(flying[g]))
                te.complete(tok, now)                            # the copy has landed (a cancel of an in-flight transfer waits for this)
                flying[g].discard(tok)
                active.discard(tok)
        elif op == "cancel" and active:
            tok = rng.choice(sorted(active))
            if te.cancel(tok) == 1:                              # queued: gone at once; in flight (2): cancelled when its copy completes
                active.discard(tok)
        else:
            drain_poll()
        for g in (0, 1):
            assert te.in_flight(g) <= W
    # finish everything that is left
    for _ in range(200):
        for g in (0, 1):
            tok = te.next_to_issue(g, now)
            if tok:
                flying[g].add(tok)
            for t in sorted(flying[g]):
                te.complete(t, now)
                flying[g].discard(t)
                active.discard(t)
        drain_poll()
        if not live:
            break
    assert not live and te.queued(0) == te.queued(1) == 0 and te.in_flight(0) == te.in_flight(1) == 0
