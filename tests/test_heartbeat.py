"""Rank liveness: heartbeats through a store, failure verdicts, and the leader refusing to start a step for a dead rank (CPU only)."""
import collections
import os
import subprocess
import sys
import time

import pytest

from layerstorm_b200.runtime.heartbeat import Heartbeat, RankFailure, RankMonitor
from layerstorm_b200.runtime.null_engine import NullEngine
from layerstorm_b200.runtime.spmd import SpmdLeader

HERE = os.path.dirname(os.path.abspath(__file__))


class DictStore:
    def __init__(self): self.d = {}
    def set(self, k, v): self.d[k] = v
    def get(self, k): return self.d[k].encode()


def test_monitor_detects_silence_and_goodbye_with_a_fake_clock():
    store, now = DictStore(), [0.0]
    hb1, hb2 = Heartbeat(store, 1), Heartbeat(store, 2)
    mon = RankMonitor(store, [1, 2, 3], timeout_s=2.0, clock=lambda: now[0])
    hb1.beat(); hb2.beat()
    assert mon.poll() == {}
    now[0] = 1.5
    hb1.beat()                                                   # rank 2 goes silent, rank 3 never showed up
    assert mon.poll() == {}
    now[0] = 2.5
    hb1.beat()
    failed = mon.poll()
    assert set(failed) == {2, 3} and "no heartbeat" in failed[2]
    with pytest.raises(RankFailure) as e:
        mon.check()
    assert e.value.ranks == [2, 3]
    hb1.stop(goodbye=True)
    assert mon.poll()[1] == "left"


def test_leader_refuses_to_announce_when_a_rank_is_down():
    store, now, q = DictStore(), [0.0], collections.deque()
    mon = RankMonitor(store, [1], timeout_s=1.0, clock=lambda: now[0])
    Heartbeat(store, 1).beat()
    mon.poll()
    lead = SpmdLeader(NullEngine(vocab=100, max_seqs=2, max_ctx=64), broadcast=q.append, monitor=mon)
    sid = lead.create_sequence()
    assert len(q) == 1
    now[0] = 5.0
    mon.poll()
    with pytest.raises(RankFailure):
        lead.prefill(sid, [1, 2, 3])
    assert len(q) == 1 and lead.seq_len(sid) == 0                # nothing announced, nothing run
    assert lead.free_page_count() > 0                            # plain reads still work


def test_background_threads_and_a_real_store():
    import torch.distributed as dist
    store = dist.HashStore()
    hb = Heartbeat(store, 1, interval_s=0.05).start()
    mon = RankMonitor(store, [1], timeout_s=0.4).start(interval_s=0.05)
    time.sleep(0.3)
    assert not mon.failed and hb.beats >= 3
    hb.stop(goodbye=False)                                       # dies without a word
    deadline = time.time() + 5
    while not mon.failed and time.time() < deadline:
        time.sleep(0.05)
    mon.stop()
    assert 1 in mon.failed and "no heartbeat" in mon.failed[1]


def test_rank_exit_is_detected_across_processes():
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29577", os.path.join(HERE, "heartbeat_worker.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert "HEARTBEAT_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]
