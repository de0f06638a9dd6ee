"""ctypes bindings of the host runtime library (``liblsb200_runtime.so``, C++20, CUDA-free).

The classes here are thin handles over the native objects; all policy and bookkeeping runs
in C++ (page allocator, expert cache, placement solver, rings, statistics, tracing ...).
"""
from __future__ import annotations

import ctypes
import re
from pathlib import Path
from typing import List, Optional, Tuple

_LIB = None
_LIB_PATH = Path(__file__).resolve().parent.parent / "_lib" / "liblsb200_runtime.so"

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
