"""Host <-> device copy microbenchmark: what the expert streamer and the KV tier can expect from the link.

    python -m layerstorm_b200.utils.h2d_bench [--gpu 0] [--max-mib 256] [--streams 1,2,4] [--numa]

Measured with CUDA events on the copy stream (3 warm-up copies, median of ``--reps``), one JSON document:
  * latency of a 64-byte pinned copy, each direction;
  * bandwidth against size (4 KiB ... ``--max-mib``), pinned H2D and D2H, and pageable H2D at the largest size;
  * aggregate H2D bandwidth of 1 / 2 / 4 concurrent streams copying one expert-slot-sized buffer each (do side streams add up?);
  * H2D bandwidth while a kernel saturates HBM on the compute stream (contention of the copy engine with a memory-bound step);
  * ``--numa``: the same large copy from a buffer bound to every NUMA node the host reports (native host arena), i.e. the
    (NUMA node, GPU) matrix the placement solver's calibration wants.
Reference: bench/h2d/h2d_bench.cu (latency / bandwidth / NUMA / contention of pinned copies).
"""
from __future__ import annotations

import argparse
import json
import statistics


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpu", type=int, default=0)
    ap.add_argument("--max-mib", type=int, default=256)
    ap.add_argument("--reps", type=int, default=9)
    ap.add_argument("--streams", default="1,2,4")
    ap.add_argument("--slot-mib", type=float, default=21.0, help="size of one streamed unit (an expert slot) for the multi-stream case")
    ap.add_argument("--numa", action="store_true")
    a = ap.parse_args(argv)

    import torch

    dev = torch.device("cuda", a.gpu)
    torch.cuda.set_device(dev)
    copy_stream = torch.cuda.Stream(device=dev)

    def timed(fn, reps=a.reps, stream=copy_stream):
        for _ in range(3):
            fn()
        stream.synchronize()
        ms = []
        for _ in range(reps):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            fn()
            e1.record(stream)
            e1.synchronize()
            ms.append(e0.elapsed_time(e1))
        return statistics.median(ms)

    out = {"gpu": torch.cuda.get_device_name(dev), "method": "CUDA events on the copy stream, 3 warm-up copies, median"}
    big_n = a.max_mib << 20
    h_pin = torch.empty(big_n, dtype=torch.uint8).pin_memory()
    h_page = torch.empty(big_n, dtype=torch.uint8)
    d = torch.empty(big_n, dtype=torch.uint8, device=dev)
    with torch.cuda.stream(copy_stream):
        out["latency_us"] = {"h2d_64B": round(timed(lambda: d[:64].copy_(h_pin[:64], non_blocking=True)) * 1e3, 2),
                             "d2h_64B": round(timed(lambda: h_pin[:64].copy_(d[:64], non_blocking=True)) * 1e3, 2)}
        sizes, n = [], 4096
        while n <= big_n:
            sizes.append(n)
            n *= 4
        if sizes[-1] != big_n:
            sizes.append(big_n)
        rows = []
        for n in sizes:
            h2d = timed(lambda: d[:n].copy_(h_pin[:n], non_blocking=True))
            d2h = timed(lambda: h_pin[:n].copy_(d[:n], non_blocking=True))
            rows.append({"bytes": n, "h2d_gb_s": round(n / h2d / 1e6, 2), "d2h_gb_s": round(n / d2h / 1e6, 2)})
        out["pinned_by_size"] = rows
        pg = timed(lambda: d.copy_(h_page, non_blocking=True), reps=3)
        out["pageable_h2d_gb_s_at_max"] = round(big_n / pg / 1e6, 2)

    # several side streams, one slot-sized copy each
    slot = int(a.slot_mib * (1 << 20))
    multi = []
    for ns in [int(x) for x in a.streams.split(",") if x.strip()]:
        streams = [torch.cuda.Stream(device=dev) for _ in range(ns)]
        hs = [torch.empty(slot, dtype=torch.uint8).pin_memory() for _ in range(ns)]
        ds = [torch.empty(slot, dtype=torch.uint8, device=dev) for _ in range(ns)]
        ms = []
        for it in range(3 + a.reps):
            torch.cuda.synchronize(dev)
            gate = torch.cuda.Event()
            gate.record()
            starts, ends = [], []
            for s, h, dd in zip(streams, hs, ds):
                s.wait_event(gate)
                with torch.cuda.stream(s):
                    b, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    b.record(s)
                    dd.copy_(h, non_blocking=True)
                    e.record(s)
                    starts.append(b)
                    ends.append(e)
            torch.cuda.synchronize(dev)
            if it >= 3:
                # first start to last end: the start events sit on the copy streams themselves, so the time the host needs to
                # reach the first copy after the synchronize is not counted
                ms.append(max(b.elapsed_time(e) for b in starts for e in ends))
        t = statistics.median(ms)
        multi.append({"streams": ns, "aggregate_h2d_gb_s": round(ns * slot / t / 1e6, 2), "ms": round(t, 3)})
    out["concurrent_streams"] = {"bytes_per_stream": slot, "rows": multi}

    # copy engine against a memory-bound kernel on the compute stream
    work = torch.empty(1 << 30, dtype=torch.uint8, device=dev)
    with torch.cuda.stream(copy_stream):
        alone = timed(lambda: d.copy_(h_pin, non_blocking=True))
    ms = []
    for it in range(3 + a.reps):
        torch.cuda.synchronize(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for _ in range(6):
            work.add_(1)
        with torch.cuda.stream(copy_stream):
            e0.record(copy_stream)
            d.copy_(h_pin, non_blocking=True)
            e1.record(copy_stream)
        torch.cuda.synchronize(dev)
        if it >= 3:
            ms.append(e0.elapsed_time(e1))
    out["contention_with_hbm_bound_kernel"] = {"h2d_gb_s_alone": round(big_n / alone / 1e6, 2),
                                               "h2d_gb_s_while_kernel_runs": round(big_n / statistics.median(ms) / 1e6, 2)}
    del work

    if a.numa:
        from ..runtime import native as rt
        per = []
        try:
            nodes = [int(t["id"]) for t in rt.numa_topology()]
        except Exception as e:                                 # no topology information on this host
            nodes, out["numa_note"] = [], f"topology unavailable: {e}"
        for node in nodes:
            try:
                arena = rt.HostArena(big_n, 1, numa_node=node)
                if not arena.pin():
                    raise OSError("cudaHostRegister refused the slab")
                buf = arena.tensor()[0]
                with torch.cuda.stream(copy_stream):
                    t = timed(lambda: d.copy_(buf, non_blocking=True))
                per.append({"numa_node": node, "bound": bool(arena.numa_bound), "h2d_gb_s": round(big_n / t / 1e6, 2)})
                arena.unpin()
            except Exception as e:
                per.append({"numa_node": node, "error": str(e)[:120]})
        out["numa_matrix"] = per
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
