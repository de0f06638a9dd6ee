"""CPU worker (gloo, one process per rank): the leader drives its engine through SpmdLeader, the followers replay the call stream;
afterwards every rank holds the same sequences."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from layerstorm_b200.runtime.null_engine import NullEngine
from layerstorm_b200.runtime.spmd import SpmdLeader, control_group, follower_loop


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo")
    grp = control_group()
    eng = NullEngine(vocab=300, max_seqs=4, max_ctx=256, page=16)
    if rank == 0:
        lead = SpmdLeader(eng, grp)
        a = lead.create_sequence()
        t = lead.prefill(a, [5, 6, 7, 8, 9])
        for _ in range(4):
            t = lead.decode([a], [t])[0]
        b = lead.fork_sequence(a)
        lead.decode([a, b], [t, t])
        lead.free_sequence(b)
        assert lead.seq_len(a) == eng.seq_len(a)                 # plain reads are not announced
        n_calls = lead.calls_announced
        lead.shutdown()
    else:
        n_calls = follower_loop(eng, grp)
    state = [None] * world
    dist.all_gather_object(state, (sorted(eng.seqs), [eng.seq_len(s) for s in sorted(eng.seqs)], n_calls))
    ok = all(s == state[0] for s in state) and state[0][2] == 9
    if rank == 0:
        print("SPMD_OK" if ok else f"SPMD_FAIL {state}", flush=True)
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
