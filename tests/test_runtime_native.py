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
