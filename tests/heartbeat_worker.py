"""CPU worker (gloo): rank 1 replays two calls, then stops beating and leaves between steps without a goodbye; the leader's monitor
notices and the next mirrored call raises RankFailure instead of being announced."""
import os
import sys
import time

import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from layerstorm_b200.runtime.heartbeat import Heartbeat, RankFailure, RankMonitor
from layerstorm_b200.runtime.null_engine import NullEngine
from layerstorm_b200.runtime.spmd import SpmdLeader, control_group, follower_loop


def main():
    rank = int(os.environ["RANK"])
    store = dist.TCPStore("127.0.0.1", int(os.environ["MASTER_PORT"]) + 1, 2, rank == 0, timeout=__import__("datetime").timedelta(seconds=60))
    dist.init_process_group("gloo")
    grp = control_group()
    eng = NullEngine(vocab=100, max_seqs=2, max_ctx=64)
    hb = Heartbeat(store, rank, interval_s=0.1).start()
    if rank == 0:
        mon = RankMonitor(store, [1], timeout_s=1.0).start(interval_s=0.1)
        lead = SpmdLeader(eng, grp, monitor=mon)
        sid = lead.create_sequence()
        lead.prefill(sid, [3, 4, 5])
        lead.shutdown()                                           # the follower leaves its loop: no call is in flight when it exits
        deadline = time.time() + 20
        while not mon.failed and time.time() < deadline:
            time.sleep(0.1)
        try:
            lead.decode([sid], [7])
            ok = False
        except RankFailure as e:
            ok = e.ranks == [1] and "no heartbeat" in str(e) and eng.seq_len(sid) == 3
        mon.stop()
        hb.stop()
        print("HEARTBEAT_OK" if ok else "HEARTBEAT_FAIL", flush=True)
    else:
        n = follower_loop(eng, grp)
        hb.stop(goodbye=False)                                    # crash-like: the counter just stops
        assert n == 2
        time.sleep(3.0)                                           # keep the store connection alive while the leader reaches its verdict
    sys.exit(0)


if __name__ == "__main__":
    main()
