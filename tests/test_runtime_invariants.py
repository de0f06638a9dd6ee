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
