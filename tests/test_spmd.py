"""SPMD command stream: in-process replay and a 2-process gloo run on the null engine (CPU only)."""
import collections
import os
import subprocess
import sys

from layerstorm_b200.runtime.null_engine import NullEngine
from layerstorm_b200.runtime.spmd import MIRRORED, SpmdLeader, follower_loop

HERE = os.path.dirname(os.path.abspath(__file__))


def test_leader_announces_and_follower_replays_in_process():
    q = collections.deque()
    lead_eng, foll_eng = NullEngine(vocab=200, max_seqs=4, max_ctx=128), NullEngine(vocab=200, max_seqs=4, max_ctx=128)
    lead = SpmdLeader(lead_eng, broadcast=q.append)
    sid = lead.create_sequence()
    tok = lead.prefill(sid, [1, 2, 3])
    out = lead.decode([sid], [tok])
    assert lead.seq_len(sid) == 4 and len(q) == 3 and [c[0] for c in q] == ["create_sequence", "prefill", "decode"]
    lead.shutdown()
    n = follower_loop(foll_eng, receive=q.popleft)
    assert n == 3 and foll_eng.seq_len(sid) == 4
    assert foll_eng.decode([sid], out) == lead_eng.decode([sid], out)         # same state -> same next token
    assert "decode" in MIRRORED and "seq_len" not in MIRRORED


def test_two_process_command_stream():
    env = dict(os.environ)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29571", os.path.join(HERE, "spmd_worker.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env)
    assert "SPMD_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]


def test_follower_reports_mirrored_failures_and_keeps_going():
    q = collections.deque()
    eng_l, eng_f = NullEngine(vocab=100, max_seqs=2, max_ctx=64), NullEngine(vocab=100, max_seqs=2, max_ctx=64)
    lead = SpmdLeader(eng_l, broadcast=q.append)
    sid = lead.create_sequence()
    try:
        lead.free_sequence(sid + 7)                       # fails on the leader ...
        raised = False
    except Exception:
        raised = True
    lead.prefill(sid, [1, 2])
    lead.shutdown()
    seen = []
    n = follower_loop(eng_f, receive=q.popleft, on_error=lambda name, e: seen.append(name))
    assert raised and seen == ["free_sequence"] and n == 3 and eng_f.seq_len(sid) == 2     # ... and the same way on the follower
