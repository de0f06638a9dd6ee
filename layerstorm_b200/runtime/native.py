"""ctypes bindings of the host runtime library (``liblsb200_runtime.so``, C++20, CUDA-free).

The classes here are thin handles over the native objects; all policy and bookkeeping runs
in C++ (page allocator, expert cache, placement solver, rings, statistics, tracing ...).
"""
from __future__ import annotations

import ctypes
import os
import re
from pathlib import Path
from typing import List, Optional, Tuple

_LIB = None
# LSB200_RUNTIME_LIB: another build of the runtime library (the sanitized one of ``build.build_sanitized``)
_LIB_PATH = Path(os.environ.get("LSB200_RUNTIME_LIB") or Path(__file__).resolve().parent.parent / "_lib" / "liblsb200_runtime.so")

OK, ERR_ARG, ERR_NOT_FOUND, ERR_EXISTS, ERR_POOL_EXHAUSTED, ERR_FROZEN, ERR_SHARED, ERR_FULL, ERR_BUSY, ERR_IO, ERR_FORMAT = range(0, -11, -1)
ERR_NAMES = {ERR_ARG: "bad argument", ERR_NOT_FOUND: "not found", ERR_EXISTS: "exists", ERR_POOL_EXHAUSTED: "kv pool exhausted",
             ERR_FROZEN: "sequence frozen", ERR_SHARED: "pages shared", ERR_FULL: "full", ERR_BUSY: "busy", ERR_IO: "io error",
             ERR_FORMAT: "bad format"}

_DECL = re.compile(r'LSB_RT_API\s+([\w\s\*:]+?)\s+(lsb_\w+)\s*\(([^)]*)\)', re.S)
_CT = {"int": ctypes.c_int, "void": None, "unsigned int": ctypes.c_uint, "char": ctypes.c_char, "bool": ctypes.c_bool, "long long": ctypes.c_longlong, "unsigned long long": ctypes.c_ulonglong,
       "float": ctypes.c_float, "double": ctypes.c_double, "uint64_t": ctypes.c_uint64, "int64_t": ctypes.c_int64,
       "uint32_t": ctypes.c_uint32, "size_t": ctypes.c_size_t}


def _ctype(decl: str):
    d = decl.replace("const", "").strip()
    if "*" in d or "ResidencyCb" in d or "Cb" in d.split()[0]:
        return ctypes.c_void_p
    for k in sorted(_CT, key=len, reverse=True):
        if d.startswith(k):
            return _CT[k]
    raise RuntimeError(f"unparsed type {decl!r}")


def load():
    """Load the library and derive every function's ctypes signature from the C++ sources."""
    global _LIB
    if _LIB is not None:
        return _LIB
    if not _LIB_PATH.exists():
        raise RuntimeError(f"native runtime library not built: {_LIB_PATH} (run `python -m layerstorm_b200.build`)")
    lib = ctypes.CDLL(str(_LIB_PATH))
    src = Path(__file__).resolve().parent.parent / "csrc" / "runtime"
    for f in sorted(src.glob("*.cpp")):
        for ret, name, params in _DECL.findall(f.read_text()):
            fn = getattr(lib, name, None)
            if fn is None:
                continue
            plist = [p.strip() for p in params.split(",") if p.strip() and p.strip() != "void"]
            fn.argtypes = [_ctype(p) for p in plist]
            fn.restype = _ctype(ret)
    _LIB = lib
    return lib


class NativeError(RuntimeError):
    def __init__(self, code: int, what: str = ""):
        super().__init__(f"{what}: {ERR_NAMES.get(code, code)}")
        self.code = code


class KvPoolExhausted(NativeError):
    pass


def _check(rc: int, what: str = ""):
    if rc == ERR_POOL_EXHAUSTED:
        raise KvPoolExhausted(rc, what)
    if rc < 0:
        raise NativeError(rc, what)
    return rc


POOL_MAIN, POOL_SPECULATION, POOL_INDEXER_K, POOL_HCA, POOL_SWA, POOL_KDA_STATE = range(6)


class PageAllocator:
    """Paged KV bookkeeping (see csrc/runtime/page_allocator.cpp)."""

    def __init__(self, pages_per_pool: List[int], page_tokens: int):
        self.lib = load()
        arr = (ctypes.c_int * len(pages_per_pool))(*pages_per_pool)
        self.h = self.lib.lsb_pa_create(len(pages_per_pool), ctypes.cast(arr, ctypes.c_void_p), page_tokens)
        self.page_tokens = page_tokens

    def __del__(self):
        if getattr(self, "h", None):
            self.lib.lsb_pa_destroy(self.h)
            self.h = None

    def free_pages(self, pool=0): return self.lib.lsb_pa_free_pages(self.h, pool)
    def total_pages(self, pool=0): return self.lib.lsb_pa_total_pages(self.h, pool)
    def lent_pages(self, pool=0): return self.lib.lsb_pa_lent_pages(self.h, pool)
    def set_headroom(self, pool, pages): self.lib.lsb_pa_set_headroom(self.h, pool, pages)
    def create(self, seq, pool=0, reserve_tokens=0): _check(self.lib.lsb_pa_seq_create(self.h, seq, pool, reserve_tokens), "seq_create")

    def extend(self, seq: int, new_len: int, privileged: bool = False) -> List[int]:
        cap = 64 + new_len // self.page_tokens
        buf = (ctypes.c_int * cap)()
        n = ctypes.c_int(0)
        _check(self.lib.lsb_pa_seq_extend(self.h, seq, new_len, int(privileged), ctypes.cast(buf, ctypes.c_void_p), cap,
                                          ctypes.cast(ctypes.pointer(n), ctypes.c_void_p)), "seq_extend")
        return list(buf[: n.value])

    def cow_frontier(self, seq: int) -> Optional[Tuple[int, int]]:
        a, b = ctypes.c_int(0), ctypes.c_int(0)
        rc = _check(self.lib.lsb_pa_cow_frontier(self.h, seq, ctypes.cast(ctypes.pointer(a), ctypes.c_void_p),
                                                 ctypes.cast(ctypes.pointer(b), ctypes.c_void_p)), "cow_frontier")
        return (a.value, b.value) if rc == 1 else None

    def fork(self, parent, child, prefix_len, frozen=False): _check(self.lib.lsb_pa_fork(self.h, parent, child, prefix_len, int(frozen)), "fork")
    def rewind(self, seq, new_len): _check(self.lib.lsb_pa_rewind(self.h, seq, new_len), "rewind")
    def destroy(self, seq): _check(self.lib.lsb_pa_seq_destroy(self.h, seq), "seq_destroy")
    def promote(self, seq, to_pool): _check(self.lib.lsb_pa_promote(self.h, seq, to_pool), "promote")
    def length(self, seq): return self.lib.lsb_pa_seq_length(self.h, seq)
    def swap_out(self, seq, idx) -> int: return _check(self.lib.lsb_pa_swap_out(self.h, seq, idx), "swap_out")
    def swap_in(self, seq, idx) -> int: return _check(self.lib.lsb_pa_swap_in(self.h, seq, idx), "swap_in")

    def pages(self, seq: int) -> List[int]:
        cap = 1 << 16
        buf = (ctypes.c_int * cap)()
        n = self.lib.lsb_pa_seq_pages(self.h, seq, ctypes.cast(buf, ctypes.c_void_p), cap)
        if n < 0:
            raise NativeError(ERR_NOT_FOUND, "seq_pages")
        return list(buf[:n])

    def refcount(self, pool, page): return self.lib.lsb_pa_refcount(self.h, pool, page)
    def claim_zone(self, pool, n): return self.lib.lsb_pa_claim_zone(self.h, pool, n)
    def release_zone(self, pool, start, n): _check(self.lib.lsb_pa_release_zone(self.h, pool, start, n), "release_zone")


def dcp_rank_for_token(token: int, chunk_tokens: int, ranks: int) -> int:
    return load().lsb_dcp_rank_for_token(token, chunk_tokens, ranks)


def dcp_local_index(token: int, chunk_tokens: int, ranks: int) -> int:
    return load().lsb_dcp_local_index(token, chunk_tokens, ranks)


ZONE_STABLE, ZONE_STREAMING = 0, 1
SLOT_FREE, SLOT_RESERVED, SLOT_READY = 0, 1, 2
POLICY = {"impact_weighted_lru": 0, "lru": 1, "lfu": 2}


class ExpertCache:
    """Two-zone fixed-slot VRAM expert cache bookkeeping (see csrc/runtime/expert_cache.cpp)."""

    def __init__(self, stable_slots: int, streaming_slots: int = 0, policy: str = "impact_weighted_lru"):
        self.lib = load()
        self.h = self.lib.lsb_ec_create(stable_slots, streaming_slots, POLICY[policy])
        self._cb = None

    def __del__(self):
        if getattr(self, "h", None):
            self.lib.lsb_ec_destroy(self.h)
            self.h = None

    def lookup(self, layer, expert): return self.lib.lsb_ec_lookup(self.h, layer, expert)
    def is_ready(self, layer, expert): return bool(self.lib.lsb_ec_is_ready(self.h, layer, expert))
    def reserve(self, layer, expert, zone=ZONE_STABLE, fallback=False): return _check(self.lib.lsb_ec_reserve(self.h, layer, expert, zone, int(fallback)), "reserve")
    def mark_ready(self, layer, expert): return _check(self.lib.lsb_ec_mark_ready(self.h, layer, expert), "mark_ready")
    def cancel(self, layer, expert): _check(self.lib.lsb_ec_cancel(self.h, layer, expert), "cancel")
    def lock(self, layer, expert): return _check(self.lib.lsb_ec_lock(self.h, layer, expert), "lock")
    def unlock(self, layer, expert): _check(self.lib.lsb_ec_unlock(self.h, layer, expert), "unlock")
    def touch(self, layer, expert, weight=0.0): self.lib.lsb_ec_touch(self.h, layer, expert, float(weight))
    def evict(self, layer, expert): return _check(self.lib.lsb_ec_evict(self.h, layer, expert), "evict")

    def pick_victim(self, zone=-1, duplicate_flags: Optional[bytes] = None):
        a, b = ctypes.c_int(0), ctypes.c_int(0)
        dup = ctypes.cast(ctypes.c_char_p(duplicate_flags), ctypes.c_void_p) if duplicate_flags else None
        s = self.lib.lsb_ec_pick_victim(self.h, zone, dup, len(duplicate_flags) if duplicate_flags else 0,
                                        ctypes.cast(ctypes.pointer(a), ctypes.c_void_p), ctypes.cast(ctypes.pointer(b), ctypes.c_void_p))
        return None if s < 0 else (s, a.value, b.value)

    def move_zone(self, layer, expert, zone): return _check(self.lib.lsb_ec_move_zone(self.h, layer, expert, zone), "move_zone")
    def add_elastic_zone(self, n): return self.lib.lsb_ec_add_elastic_zone(self.h, n)
    def remove_elastic_zone(self, gen): _check(self.lib.lsb_ec_remove_elastic_zone(self.h, gen), "remove_elastic_zone")
    def generation(self): return self.lib.lsb_ec_generation(self.h)
    def n_slots(self): return self.lib.lsb_ec_n_slots(self.h)
    def count(self, zone=-1, state=SLOT_READY): return self.lib.lsb_ec_count(self.h, zone, state)

    def slot_info(self, slot):
        v = [ctypes.c_int(0) for _ in range(5)]
        _check(self.lib.lsb_ec_slot_info(self.h, slot, *[ctypes.cast(ctypes.pointer(x), ctypes.c_void_p) for x in v]), "slot_info")
        return dict(zip(("state", "zone", "layer", "expert", "locks"), (x.value for x in v)))

    WEIGHT_FIELDS = ("eviction_alpha_recency", "eviction_beta_frequency", "eviction_gamma_routing_weight", "eviction_delta_temporal_autocorr",
                     "eviction_epsilon_coactivation", "eviction_zeta_prefetch_score", "eviction_eta_hysteresis")

    def set_weights(self, policy: str, weights):
        """Policy + the seven score weights (alpha .. eta); may be called at any time (configuration hot reload)."""
        w = (ctypes.c_float * 7)(*[float(x) for x in weights])
        self.lib.lsb_ec_set_weights(self.h, POLICY[policy], ctypes.cast(w, ctypes.c_void_p))

    def configure(self, section: dict):
        """``section`` = the ``memory.expert_cache`` configuration section."""
        self.set_weights(section.get("eviction_policy", "impact_weighted_lru"), [section.get(k, 0.0) for k in self.WEIGHT_FIELDS])

    def set_hysteresis(self, stages=5, up=5, down=1, window_steps=16, ema=0.1):
        self.lib.lsb_ec_set_hysteresis(self.h, stages, up, down, window_steps, float(ema))

    def set_hint(self, layer, expert, coactivation=-1.0, prefetch_score=-1.0):
        return self.lib.lsb_ec_set_hint(self.h, layer, expert, float(coactivation), float(prefetch_score)) == 0

    def end_step(self): self.lib.lsb_ec_end_step(self.h)

    def slot_stats(self, slot):
        out = (ctypes.c_float * 7)()
        _check(self.lib.lsb_ec_slot_stats(self.h, slot, ctypes.cast(out, ctypes.c_void_p)), "slot_stats")
        return dict(zip(("recency", "frequency", "routing_weight", "temporal_autocorr", "coactivation", "prefetch_score", "hysteresis"), out))

    def set_listener(self, fn):
        CB = ctypes.CFUNCTYPE(None, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int)
        self._cb = CB(lambda user, layer, expert, slot, resident: fn(layer, expert, slot, bool(resident)))
        self.lib.lsb_ec_set_listener(self.h, ctypes.cast(self._cb, ctypes.c_void_p), None)


def _vp(x):
    return ctypes.cast(x, ctypes.c_void_p)


def _iarr(vals, ct=ctypes.c_int):
    return (ct * len(vals))(*vals)


class ExpertStats:
    def __init__(self, n: int, alpha: float = 0.05):
        self.lib, self.n = load(), n
        self.h = self.lib.lsb_es_create(n, alpha)

    def __del__(self):
        if getattr(self, "h", None):
            self.lib.lsb_es_destroy(self.h); self.h = None

    def observe(self, ids, weights=None):
        a = _iarr(list(ids))
        w = _iarr(list(weights), ctypes.c_float) if weights is not None else None
        self.lib.lsb_es_observe(self.h, _vp(a), _vp(w) if w is not None else None, len(ids))

    def frequency(self, e): return self.lib.lsb_es_frequency(self.h, e)
    def weight(self, e): return self.lib.lsb_es_weight(self.h, e)
    def autocorr(self, e): return self.lib.lsb_es_autocorr(self.h, e)
    def recency(self, e): return self.lib.lsb_es_recency(self.h, e)

    def frequencies(self):
        out = (ctypes.c_float * self.n)()
        self.lib.lsb_es_frequencies(self.h, _vp(out))
        return list(out)


class CoactivationGraph:
    def __init__(self, n: int, decay: float = 0.99):
        self.lib, self.n = load(), n
        self.h = self.lib.lsb_cg_create(n, decay)

    def __del__(self):
        if getattr(self, "h", None):
            self.lib.lsb_cg_destroy(self.h); self.h = None

    def observe(self, ids): self.lib.lsb_cg_observe(self.h, _vp(_iarr(list(ids))), len(ids))
    def weight(self, a, b): return self.lib.lsb_cg_weight(self.h, a, b)

    def partition(self, parts: int):
        out = (ctypes.c_int * self.n)()
        self.lib.lsb_cg_partition(self.h, parts, _vp(out))
        return list(out)


class WorkloadDetector:
    def __init__(self, n: int, window: int = 256, z: float = 4.0):
        self.lib = load()
        self.h = self.lib.lsb_wd_create(n, window, z)

    def __del__(self):
        if getattr(self, "h", None):
            self.lib.lsb_wd_destroy(self.h); self.h = None

    def observe(self, freq) -> bool: return bool(self.lib.lsb_wd_observe(self.h, _vp(_iarr(list(freq), ctypes.c_float))))
    def shifts(self): return self.lib.lsb_wd_shifts(self.h)


class AcceptanceTracker:
    def __init__(self, alpha: float = 0.1, window: int = 64):
        self.lib = load()
        self.h = self.lib.lsb_at_create(alpha, window)

    def __del__(self):
        if getattr(self, "h", None):
            self.lib.lsb_at_destroy(self.h); self.h = None

    def record(self, request, proposed, accepted): self.lib.lsb_at_record(self.h, request, proposed, accepted)
    def ema(self): return self.lib.lsb_at_ema(self.h)
    def global_rate(self): return self.lib.lsb_at_global(self.h)
    def windowed_rate(self): return self.lib.lsb_at_windowed(self.h)
    def request_rate(self, r): return self.lib.lsb_at_request(self.h, r)
    def forget(self, r): self.lib.lsb_at_forget(self.h, r)
    def expected_tokens(self, gamma): return self.lib.lsb_at_expected_tokens(self.h, gamma)


class SpscRing:
    """Lock-free single-producer/single-consumer ring of fixed-size slots (power-of-two capacity)."""

    def __init__(self, slots: int, slot_bytes: int):
        self.lib, self.slot_bytes = load(), slot_bytes
        self.h = self.lib.lsb_ring_create(slots, slot_bytes)
        if not self.h:
            raise ValueError("ring capacity must be a power of two")

    def __del__(self):
        if getattr(self, "h", None):
            self.lib.lsb_ring_destroy(self.h); self.h = None

    def push(self, data: bytes) -> bool: return bool(self.lib.lsb_ring_push(self.h, ctypes.c_char_p(data), len(data)))

    def pop(self) -> Optional[bytes]:
        buf = ctypes.create_string_buffer(self.slot_bytes)
        return buf.raw if self.lib.lsb_ring_pop(self.h, _vp(buf)) else None

    def __len__(self): return int(self.lib.lsb_ring_size(self.h))


class StateSnapshot:
    """Seqlock-published state block: one writer, any number of wait-free readers."""

    def __init__(self, nbytes: int):
        self.lib, self.nbytes = load(), nbytes
        self.h = self.lib.lsb_snap_create(nbytes)

    def __del__(self):
        if getattr(self, "h", None):
            self.lib.lsb_snap_destroy(self.h); self.h = None

    def begin(self): self.lib.lsb_snap_begin(self.h)
    def write(self, off: int, data: bytes): self.lib.lsb_snap_write(self.h, off, ctypes.c_char_p(data), len(data))
    def end(self): self.lib.lsb_snap_end(self.h)

    def read(self, off: int, n: int, tries: int = 64):
        buf = ctypes.create_string_buffer(n)
        v = self.lib.lsb_snap_read(self.h, _vp(buf), off, n, tries)
        return (buf.raw, int(v)) if v else (None, 0)


class PerfTrace:
    """Preallocated ring of 32-byte trace records (see csrc/runtime/ipc.cpp)."""

    def __init__(self, capacity: int = 1 << 20):
        self.lib = load()
        self.h = self.lib.lsb_trace_create(capacity)

    def __del__(self):
        if getattr(self, "h", None):
            self.lib.lsb_trace_destroy(self.h); self.h = None

    def record(self, stage, gpu=0, cmd_seq=0, key=0, token=0): self.lib.lsb_trace_record(self.h, stage, gpu, cmd_seq, key, token)
    def count(self): return int(self.lib.lsb_trace_count(self.h))
    def dropped(self): return int(self.lib.lsb_trace_dropped(self.h))
    def dump_csv(self, path): _check(self.lib.lsb_trace_dump_csv(self.h, path.encode()), "dump_csv")

    def span_ns(self, begin_stage, end_stage):
        n = ctypes.c_ulonglong(0)
        t = self.lib.lsb_trace_span_ns(self.h, begin_stage, end_stage, _vp(ctypes.pointer(n)))
        return int(t), int(n.value)


class LoaderSolver:
    """Expert placement solver (see csrc/runtime/loader_solver.cpp).  rates in bytes/us, times in ns."""

    def __init__(self, a_ns, b_ns, rate_bpus, lat_ns, egress_bpus, batch_p=64, recon_ns=0, evict_ns=0):
        self.lib = load()
        self.M, self.B = len(a_ns), len(egress_bpus)
        LL = ctypes.c_longlong
        flat = lambda m: [x for row in m for x in row]
        self.h = self.lib.lsb_solver_create(self.M, self.B, batch_p, _vp(_iarr(a_ns, LL)), _vp(_iarr(b_ns, LL)), _vp(_iarr(flat(rate_bpus), LL)),
                                            _vp(_iarr(flat(lat_ns), LL)), _vp(_iarr(egress_bpus, LL)), recon_ns, evict_ns)

    def __del__(self):
        if getattr(self, "h", None):
            self.lib.lsb_solver_destroy(self.h); self.h = None

    def _req(self, bank, nbytes, resident, free_slots):
        n = len(bank)
        res = (ctypes.c_ubyte * (n * self.M))(*[int(resident[e][m]) for e in range(n) for m in range(self.M)])
        return n, _iarr(bank), _iarr(nbytes, ctypes.c_longlong), res, _iarr(free_slots)

    def solve(self, bank, nbytes, resident, free_slots, tier=0):
        n, b, by, res, fs = self._req(bank, nbytes, resident, free_slots)
        out = (ctypes.c_int * n)()
        cost = ctypes.c_longlong(0)
        used = _check(self.lib.lsb_solver_solve(self.h, n, _vp(b), _vp(by), _vp(res), _vp(fs), tier, _vp(out), _vp(ctypes.pointer(cost))), "solve")
        return list(out), int(cost.value), used

    def evaluate(self, bank, nbytes, resident, free_slots, assign):
        n, b, by, res, fs = self._req(bank, nbytes, resident, free_slots)
        return int(self.lib.lsb_solver_evaluate(self.h, n, _vp(b), _vp(by), _vp(res), _vp(fs), _vp(_iarr(assign))))


def _out(ct=ctypes.c_int):
    v = ct(0)
    return v, _vp(ctypes.pointer(v))


class TransferEngine:
    """Queueing / de-duplication / priority core of the async transfer engine (csrc/runtime/transfer_engine.cpp).
    dir 0 = host->device, 1 = device->host.  States: 0 queued, 1 in flight, 2 done, 3 cancelled."""
    H2D, D2H = 0, 1

    def __init__(self, n_gpus: int = 1, levels: int = 3, waterline: int = 4):
        self.lib = load()
        self.h = self.lib.lsb_te_create(n_gpus, levels, waterline)

    def __del__(self):
        if getattr(self, "h", None):
            self.lib.lsb_te_destroy(self.h); self.h = None

    def submit(self, layer, expert, gpu=0, direction=0, priority=0, nbytes=0) -> int:
        return int(self.lib.lsb_te_submit(self.h, layer, expert, gpu, direction, priority, nbytes))

    def next_to_issue(self, gpu=0, now_ns=0) -> int: return int(self.lib.lsb_te_next(self.h, gpu, now_ns))

    def info(self, token):
        vals = [_out() for _ in range(5)]
        b, bp = _out(ctypes.c_longlong)
        st, stp = _out()
        _check(self.lib.lsb_te_info(self.h, token, *(p for _, p in vals), bp, stp), "transfer info")
        l, e, g, d, pr = (v.value for v, _ in vals)
        return {"layer": l, "expert": e, "gpu": g, "dir": d, "priority": pr, "bytes": b.value, "state": st.value}

    def complete(self, token, now_ns=0): _check(self.lib.lsb_te_complete(self.h, token, now_ns), "transfer complete")
    def cancel(self, token) -> int: return _check(self.lib.lsb_te_cancel(self.h, token), "transfer cancel")

    def poll(self, cap: int = 64):
        toks = (ctypes.c_ulonglong * cap)()
        arrs = [(ctypes.c_int * cap)() for _ in range(4)]
        n = self.lib.lsb_te_poll(self.h, _vp(toks), *(_vp(a) for a in arrs), cap)
        return [(int(toks[i]), arrs[0][i], arrs[1][i], arrs[2][i], arrs[3][i]) for i in range(n)]      # token, state, layer, expert, gpu

    def queued(self, gpu=0): return self.lib.lsb_te_queued(self.h, gpu)
    def in_flight(self, gpu=0): return self.lib.lsb_te_in_flight(self.h, gpu)
    def bandwidth_gbs(self, gpu=0, direction=0): return self.lib.lsb_te_bandwidth_gbs(self.h, gpu, direction)
    def dedup_hits(self): return int(self.lib.lsb_te_dedup_hits(self.h))
    def find(self, layer, expert, gpu=0, direction=0): return int(self.lib.lsb_te_find(self.h, layer, expert, gpu, direction))


def numa_topology(sysfs_root: str = ""):
    lib = load()
    cap = 64
    ids, cpus = (ctypes.c_int * cap)(), (ctypes.c_int * cap)()
    tot, free = (ctypes.c_longlong * cap)(), (ctypes.c_longlong * cap)()
    n = min(cap, lib.lsb_numa_topology(sysfs_root.encode(), cap, _vp(ids), _vp(tot), _vp(free), _vp(cpus)))
    return [{"id": ids[i], "total_bytes": tot[i], "free_bytes": free[i], "n_cpus": cpus[i]} for i in range(n)]


SIZING_MODES = {"fraction_free": 0, "fraction_total": 1, "absolute_gb": 2}


def host_pool_budget(mode: str, value: float, total_bytes: int, free_bytes: int, reserve_bytes: int = 0) -> int:
    return int(load().lsb_host_pool_budget(SIZING_MODES[mode], value, total_bytes, free_bytes, reserve_bytes))


class HostArena:
    """Slotted host slab for expert weights (csrc/runtime/host_arena.cpp).  ``tensor()`` exposes the slab as a
    uint8 torch tensor without copying; ``pin()`` registers it with the CUDA driver."""
    EMPTY, LOADING, ACTIVE = 0, 1, 2

    def __init__(self, slot_bytes: int, n_slots: int, numa_node: int = -1, memfd: bool = False, thp: bool = True, attach_fd: int = -1):
        self.lib = load()
        self.slot_bytes, self.n_slots = slot_bytes, n_slots
        if attach_fd >= 0:
            self.h = self.lib.lsb_arena_attach(slot_bytes, n_slots, attach_fd)
        else:
            self.h = self.lib.lsb_arena_create(slot_bytes, n_slots, numa_node, int(memfd), int(thp))
        if not self.h:
            raise MemoryError(f"cannot map a host arena of {slot_bytes * n_slots} bytes")
        self._tensor = None
        self._pinned = False

    def __del__(self):
        if getattr(self, "h", None):
            self.unpin()
            self._tensor = None
            self.lib.lsb_arena_destroy(self.h); self.h = None

    @property
    def base(self) -> int: return int(self.lib.lsb_arena_base(self.h) or 0)
    @property
    def nbytes(self) -> int: return int(self.lib.lsb_arena_bytes(self.h))
    @property
    def fd(self) -> int: return self.lib.lsb_arena_fd(self.h)
    @property
    def numa_bound(self) -> bool: return bool(self.lib.lsb_arena_numa_bound(self.h))

    def tensor(self):
        import torch
        if self._tensor is None:
            buf = (ctypes.c_uint8 * self.nbytes).from_address(self.base)
            self._tensor = torch.frombuffer(buf, dtype=torch.uint8).view(self.n_slots, self.slot_bytes)
        return self._tensor

    def pin(self) -> bool:
        """Page-lock the slab for asynchronous copies (cudaHostRegister, portable).  False without a CUDA device."""
        import torch
        if self._pinned or not torch.cuda.is_available():
            return self._pinned
        rc = torch.cuda.cudart().cudaHostRegister(self.base, self.nbytes, 1)
        self._pinned = int(rc) == 0
        return self._pinned

    def unpin(self):
        if self._pinned:
            try:
                import torch
                torch.cuda.cudart().cudaHostUnregister(self.base)
            except ImportError:          # interpreter shutdown: the driver releases the registration with the process
                pass
            self._pinned = False

    def lookup(self, layer, expert) -> int: return self.lib.lsb_arena_lookup(self.h, layer, expert)

    def begin_load(self, layer, expert):
        el, elp = _out()
        ee, eep = _out()
        slot = _check(self.lib.lsb_arena_begin_load(self.h, layer, expert, elp, eep), "arena begin_load")
        return slot, ((el.value, ee.value) if el.value >= 0 else None)

    def finish_load(self, slot, ok=True): _check(self.lib.lsb_arena_finish_load(self.h, slot, int(ok)), "arena finish_load")
    def ref(self, slot, delta=1): return _check(self.lib.lsb_arena_ref(self.h, slot, delta), "arena ref")
    def wipe(self): _check(self.lib.lsb_arena_wipe(self.h), "arena wipe")

    def stats(self):
        U = ctypes.c_ulonglong
        (a, ap), (b, bp), (c, cp) = _out(U), _out(U), _out(U)
        n, np_ = _out()
        self.lib.lsb_arena_stats(self.h, ap, bp, cp, np_)
        return {"hits": a.value, "misses": b.value, "evictions": c.value, "active": n.value}

    def slot_info(self, slot):
        vals = [_out() for _ in range(4)]
        _check(self.lib.lsb_arena_slot_info(self.h, slot, *(p for _, p in vals)), "arena slot_info")
        st, l, e, r = (v.value for v, _ in vals)
        return {"state": st, "layer": l, "expert": e, "refs": r}

    def save_meta(self, path, tag=0): _check(self.lib.lsb_arena_save_meta(self.h, str(path).encode(), tag), "arena save_meta")
    def load_meta(self, path, tag=0) -> int: return self.lib.lsb_arena_load_meta(self.h, str(path).encode(), tag)


class NvmeTier:
    def __init__(self, drives, capacity_bytes: int = 0, queue_depth: int = 64, direct_io: bool = False, workers: int = 4):
        self.lib = load()
        self.h = self.lib.lsb_nvme_create("\n".join(str(d) for d in drives).encode(), capacity_bytes, queue_depth, int(direct_io), workers)
        if not self.h:
            raise ValueError("NvmeTier needs at least one drive path")

    def __del__(self):
        if getattr(self, "h", None):
            self.lib.lsb_nvme_destroy(self.h); self.h = None

    def write(self, layer, expert, data: bytes): _check(self.lib.lsb_nvme_write(self.h, layer, expert, ctypes.c_char_p(data), len(data)), "nvme write")

    def write_ptr(self, layer, expert, ptr: int, nbytes: int): _check(self.lib.lsb_nvme_write(self.h, layer, expert, ctypes.c_void_p(ptr), nbytes), "nvme write")

    def read(self, layer, expert, nbytes: int) -> bytes:
        buf = ctypes.create_string_buffer(nbytes)
        _check(self.lib.lsb_nvme_read(self.h, layer, expert, _vp(buf), nbytes), "nvme read")
        return buf.raw

    def read_async(self, layer, expert, dst_ptr: int, nbytes: int) -> int:
        return int(self.lib.lsb_nvme_read_async(self.h, layer, expert, ctypes.c_void_p(dst_ptr), nbytes))

    def poll(self, cap=64):
        toks, st = (ctypes.c_ulonglong * cap)(), (ctypes.c_int * cap)()
        n = self.lib.lsb_nvme_poll(self.h, _vp(toks), _vp(st), cap)
        return [(int(toks[i]), st[i]) for i in range(n)]

    def size_of(self, layer, expert): return int(self.lib.lsb_nvme_size_of(self.h, layer, expert))
    def evict(self, layer, expert): _check(self.lib.lsb_nvme_evict(self.h, layer, expert), "nvme evict")
    def used(self): return int(self.lib.lsb_nvme_used(self.h))
    def pending(self): return self.lib.lsb_nvme_pending(self.h)


class ExpertLifecycle:
    """Per (layer, expert, gpu) residency state machine (csrc/runtime/lifecycle.cpp)."""
    COLD, LOADING_TO_RAM, WARM = 0, 1, 2
    ABSENT, RESERVED, TRANSFERRING, HOT, DRAINING = 0, 1, 2, 3, 4
    ACT_NONE, ACT_READ_NVME, ACT_RESERVE_SLOT, ACT_START_H2D, ACT_WAIT = 0, 1, 2, 3, 4
    (EV_NVME_DONE, EV_NVME_FAILED, EV_SLOT_RESERVED, EV_SLOT_DENIED, EV_H2D_STARTED, EV_H2D_DONE, EV_H2D_FAILED, EV_EVICT_REQUESTED,
     EV_DRAINED, EV_HOST_EVICTED) = range(10)

    def __init__(self):
        self.lib = load()
        self.h = self.lib.lsb_elm_create()

    def __del__(self):
        if getattr(self, "h", None):
            self.lib.lsb_elm_destroy(self.h); self.h = None

    def set_host_tier(self, layer, expert, tier): self.lib.lsb_elm_set_host_tier(self.h, layer, expert, tier)
    def begin_host_load(self, layer, expert): self.lib.lsb_elm_begin_host_load(self.h, layer, expert)

    def ensure_resident(self, layer, expert, gpu=0):
        t, tp = _out(ctypes.c_ulonglong)
        a = self.lib.lsb_elm_ensure_resident(self.h, layer, expert, gpu, tp)
        return a, int(t.value)

    def release(self, layer, expert, gpu=0): return self.lib.lsb_elm_release(self.h, layer, expert, gpu)
    def on_event(self, layer, expert, gpu, ev) -> int: return _check(self.lib.lsb_elm_on_event(self.h, layer, expert, gpu, ev), "lifecycle event")

    def get(self, layer, expert, gpu=0):
        vals = [_out() for _ in range(3)]
        self.lib.lsb_elm_get(self.h, layer, expert, gpu, *(p for _, p in vals))
        return tuple(v.value for v, _ in vals)          # host tier, gpu tier, interest

    def loads(self): return int(self.lib.lsb_elm_loads(self.h))
    def evictions(self): return int(self.lib.lsb_elm_evictions(self.h))


class ZoneRebalancer:
    NONE, LEND, BEGIN_RECLAIM, FINISH_RECLAIM = range(4)

    def __init__(self, total_kv_pages, pages_per_zone, low_water=0.5, high_water=0.85, max_zones=4):
        self.lib = load()
        self.h = self.lib.lsb_zr_create(total_kv_pages, pages_per_zone, low_water, high_water, max_zones)

    def __del__(self):
        if getattr(self, "h", None):
            self.lib.lsb_zr_destroy(self.h); self.h = None

    def step(self, kv_used, miss_rate, zone_occupancy=0):
        g, gp = _out()
        a = self.lib.lsb_zr_step(self.h, kv_used, miss_rate, zone_occupancy, gp)
        return a, g.value

    def on_lent(self, gen): self.lib.lsb_zr_on_lent(self.h, gen)
    def on_reclaimed(self, gen): _check(self.lib.lsb_zr_on_reclaimed(self.h, gen), "zone reclaim")
    def lent_pages(self): return self.lib.lsb_zr_lent_pages(self.h)
    def n_zones(self): return self.lib.lsb_zr_n_zones(self.h)


class KvTierTable:
    HOT_PAGE, ROW_CACHE, COLD = 0, 1, 2

    def __init__(self, page_tokens, hot_window_tokens, cold_slots, row_cache_rows=0):
        self.lib = load()
        self.h = self.lib.lsb_kvt_create(page_tokens, hot_window_tokens, cold_slots, row_cache_rows)

    def __del__(self):
        if getattr(self, "h", None):
            self.lib.lsb_kvt_destroy(self.h); self.h = None

    def create(self, seq): self.lib.lsb_kvt_seq_create(self.h, seq)
    def fork(self, parent, child, prefix_pages): _check(self.lib.lsb_kvt_seq_fork(self.h, parent, child, prefix_pages), "tier fork")
    def destroy(self, seq): _check(self.lib.lsb_kvt_seq_destroy(self.h, seq), "tier destroy")

    def demotion_candidates(self, seq, seq_len, cap=256):
        out = (ctypes.c_int * cap)()
        n = _check(self.lib.lsb_kvt_demotion_candidates(self.h, seq, seq_len, _vp(out), cap), "tier candidates")
        return list(out[:n])

    def demote(self, seq, page) -> int: return _check(self.lib.lsb_kvt_demote(self.h, seq, page), "tier demote")
    def promote(self, seq, page) -> int: return _check(self.lib.lsb_kvt_promote(self.h, seq, page), "tier promote")
    def truncate(self, seq, new_len): _check(self.lib.lsb_kvt_truncate(self.h, seq, new_len), "tier truncate")
    def where(self, seq, page) -> int: return self.lib.lsb_kvt_where(self.h, seq, page)

    def classify(self, seq, layer, rows):
        n = len(rows)
        kind, ref = (ctypes.c_int * n)(), (ctypes.c_int * n)()
        cold = _check(self.lib.lsb_kvt_classify(self.h, seq, layer, _vp(_iarr(list(rows))), n, _vp(kind), _vp(ref)), "tier classify")
        return list(kind), list(ref), cold

    def cache_row(self, seq, layer, row) -> int: return self.lib.lsb_kvt_cache_row(self.h, seq, layer, row)
    def free_cold_slots(self): return self.lib.lsb_kvt_free_cold_slots(self.h)

    def stats(self):
        U = ctypes.c_ulonglong
        vals = [_out(U) for _ in range(4)]
        self.lib.lsb_kvt_stats(self.h, *(p for _, p in vals))
        return dict(zip(("demotions", "promotions", "cold_fetches", "row_hits"), (v.value for v, _ in vals)))


VRAM_REGIONS = ("weights", "workspace", "kv_spec", "indexer_k", "kv_main", "prefill_scratch", "recurrent", "expert_streaming", "expert_stable", "safety")


def vram_plan(total_bytes, weights_bytes, workspace_bytes, kv_bytes_per_page, kv_pages, spec_pool_fraction=0.15, indexer_bytes_per_page=0,
              indexer_pages=0, prefill_scratch_bytes=0, recurrent_bytes_per_seq=0, recurrent_seqs=0, expert_slot_bytes=0,
              expert_slots_wanted=0, stable_zone_fraction=0.7, safety_bytes=1 << 30):
    """Carve one GPU (csrc/runtime/vram_planner.cpp).  Raises NativeError(ERR_FULL) naming the region that does not fit."""
    inp = (ctypes.c_double * 16)(total_bytes, weights_bytes, workspace_bytes, kv_bytes_per_page, kv_pages, spec_pool_fraction, indexer_bytes_per_page,
                                 indexer_pages, prefill_scratch_bytes, recurrent_bytes_per_seq, recurrent_seqs, expert_slot_bytes,
                                 expert_slots_wanted, stable_zone_fraction, safety_bytes, 0)
    out = (ctypes.c_longlong * 23)()
    failed = load().lsb_vram_plan(_vp(inp), _vp(out))
    if failed >= 0:
        raise NativeError(ERR_FULL, f"VRAM plan: region '{VRAM_REGIONS[failed]}' does not fit")
    regions = {VRAM_REGIONS[r]: {"offset": out[r], "size": out[10 + r]} for r in range(10)}
    return {"regions": regions, "kv_spec_pages": out[20], "expert_stable_slots": out[21], "expert_streaming_slots": out[22]}


class Determinism:
    def __init__(self):
        self.lib = load()
        self.h = self.lib.lsb_det_create()

    def __del__(self):
        if getattr(self, "h", None):
            self.lib.lsb_det_destroy(self.h); self.h = None

    def set_flags(self, deterministic=False, identity=False):
        buf = ctypes.create_string_buffer(128)
        rc = self.lib.lsb_det_set_flags(self.h, int(deterministic), int(identity), _vp(buf), 128)
        if rc < 0:
            raise NativeError(rc, f"determinism: pinned knob '{buf.value.decode()}' contradicts the requested mode")

    def pin(self, name, value): _check(self.lib.lsb_det_pin(self.h, name.encode(), int(value)), f"determinism pin {name}")
    def get(self, name) -> int: return _check(self.lib.lsb_det_get(self.h, name.encode()), f"determinism knob {name}")

    def knobs(self):
        self.lib.lsb_det_name_at.restype = ctypes.c_char_p
        return [self.lib.lsb_det_name_at(self.h, i).decode() for i in range(self.lib.lsb_det_count(self.h))]


class BufferRegistry:
    def __init__(self):
        self.lib = load()
        self.h = self.lib.lsb_bufreg_create()

    def __del__(self):
        if getattr(self, "h", None):
            self.lib.lsb_bufreg_destroy(self.h); self.h = None

    def add(self, name, ptr, nbytes, gpu=0) -> int: return _check(self.lib.lsb_bufreg_add(self.h, name.encode(), ptr, nbytes, gpu), f"buffer {name}")
    def find(self, name) -> int: return _check(self.lib.lsb_bufreg_find(self.h, name.encode()), f"buffer {name}")

    def get(self, bid):
        U = ctypes.c_ulonglong
        (p, pp), (b, bp) = _out(U), _out(U)
        g, gp = _out()
        _check(self.lib.lsb_bufreg_get(self.h, bid, pp, bp, gp), "buffer id")
        return p.value, b.value, g.value

    def contains(self, bid, ptr, nbytes) -> bool: return bool(self.lib.lsb_bufreg_contains(self.h, bid, ptr, nbytes))
    def __len__(self): return self.lib.lsb_bufreg_count(self.h)


class CpuExperts:
    """Host execution of expert FFNs from the GPU's slot images (csrc/runtime/cpu_experts.cpp)."""

    def __init__(self, threads: int = 0, cpus: Optional[List[int]] = None):
        import os
        self.lib = load()
        n = threads or max(1, min(32, os.cpu_count() or 1))
        arr = _iarr(list(cpus)) if cpus else None
        self.h = self.lib.lsb_cpu_pool_create(n, _vp(arr) if arr is not None else None, len(cpus) if cpus else 0)

    def __del__(self):
        if getattr(self, "h", None):
            self.lib.lsb_cpu_pool_destroy(self.h); self.h = None

    @property
    def threads(self) -> int: return self.lib.lsb_cpu_pool_size(self.h)

    def ffn(self, ef_struct_addr: int, slot, x, limit: float = 0.0, scale=None, out=None, accumulate: bool = False):
        """``slot``: uint8 CPU tensor (one slot image); ``x``: fp32 CPU [n, H]."""
        import torch
        x = x.contiguous().float()
        n, H = x.shape
        out = torch.zeros(n, H) if out is None else out
        sc = scale.contiguous().float() if scale is not None else None
        _check(self.lib.lsb_cpu_expert_ffn(self.h, ctypes.c_void_p(ef_struct_addr), ctypes.c_void_p(slot.data_ptr()), ctypes.c_void_p(x.data_ptr()), n,
                                           float(limit), ctypes.c_void_p(sc.data_ptr()) if sc is not None else None,
                                           ctypes.c_void_p(out.data_ptr()), int(accumulate)), "cpu expert ffn")
        return out

    def moe_layer(self, ef_struct_addr: int, slots: dict, n_experts: int, x, ids, wts, limit: float = 0.0):
        """``slots``: expert id -> uint8 CPU tensor.  Returns fp32 [tokens, H]."""
        import torch
        x, ids, wts = x.contiguous().float(), ids.contiguous().int(), wts.contiguous().float()
        T, H = x.shape
        S = ids.shape[1]
        ptrs = (ctypes.c_void_p * n_experts)(*[ctypes.c_void_p(slots[e].data_ptr()) if e in slots else None for e in range(n_experts)])
        out = torch.zeros(T, H)
        _check(self.lib.lsb_cpu_moe_layer(self.h, ctypes.c_void_p(ef_struct_addr), _vp(ptrs), n_experts, ctypes.c_void_p(x.data_ptr()),
                                          ctypes.c_void_p(ids.data_ptr()), ctypes.c_void_p(wts.data_ptr()), T, S, float(limit),
                                          ctypes.c_void_p(out.data_ptr())), "cpu moe layer")
        return out
