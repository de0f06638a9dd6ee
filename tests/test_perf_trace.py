"""Stage tracing around engine calls and the trace report (CPU, null engine)."""
import json
import os

from layerstorm_b200.runtime.null_engine import NullEngine
from layerstorm_b200.utils import perf_trace as pt


def test_traced_engine_records_spans_and_report_aggregates(tmp_path):
    tr = pt.Tracer(capacity=4096)
    eng = pt.TracedEngine(NullEngine(vocab=100, max_seqs=2, max_ctx=64), tr)
    sid = eng.create_sequence()
    tok = eng.prefill(sid, [1, 2, 3, 4, 5])
    for _ in range(7):
        tok = eng.decode([sid], [tok])[0]
    assert eng.seq_len(sid) == 12                               # untraced attribute access passes through
    eng.free_sequence(sid)
    path = str(tmp_path / "trace.csv")
    rep = tr.dump(path)
    assert rep["records"] == 2 * (1 + 1 + 7 + 1) and rep["unmatched_begins"] == 0 and rep["dropped_records"] == 0
    s = rep["spans"]
    assert s["decode"]["calls"] == 7 and s["decode"]["items"] == 7 and s["prefill"]["calls"] == 1 and s["prefill"]["items"] == 5
    assert s["decode"]["p50_us"] <= s["decode"]["p99_us"] and s["decode"]["total_ms"] >= 0
    side = json.load(open(os.path.splitext(path)[0] + ".json"))
    assert side["spans"].keys() == s.keys()
    table = pt.format_table(rep)
    assert "decode" in table and "items/s" in table
    assert pt.main(["report", path, "-o", str(tmp_path / "again.json")]) == 0


def test_env_switches():
    assert not pt.enabled({}) and not pt.enabled({"LS_PERF_TRACE": "0"}) and pt.enabled({"LS_PERF_TRACE": "1"})
    assert pt.out_path({}) == "lsb_perf_trace.csv" and pt.out_path({"LS_PERF_TRACE_OUT": "/tmp/x.csv"}) == "/tmp/x.csv"
