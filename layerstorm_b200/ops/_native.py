"""ctypes binding of ``liblsb200_kernels.so`` (the hand-written sm_100a kernels).

Every exported launcher takes raw device pointers, sizes and a CUDA stream handle and
returns a ``cudaError_t`` (0 = ok, -1 = argument rejected by the launcher).  ``call``
converts torch tensors to pointers, appends the current torch stream and raises on a
non-zero status, so a missing or broken extension fails loudly instead of silently
falling back to PyTorch.
"""
from __future__ import annotations

import ctypes
import os
import re
from pathlib import Path

import torch

_LIB = None
# LSB200_KERNELS_LIB: load another build of the kernel library (kernel tuning experiments).
_LIB_PATH = Path(os.environ.get("LSB200_KERNELS_LIB") or Path(__file__).resolve().parent.parent / "_lib" / "liblsb200_kernels.so")

# signature letters: p pointer, i int32, l int64, f float, u uint64; the trailing stream is appended.
_DECL = re.compile(r'LSB_API\s+int\s+(lsb_\w+)\s*\(([^)]*)\)', re.S)


def _parse_sigs() -> dict:
    """Derive the ctypes signatures from the ``LSB_API int lsb_*(...)`` declarations in the
    kernel sources, so the Python side can never drift from the C side."""
    sigs = {}
    src_dir = Path(__file__).resolve().parent.parent / "csrc" / "kernels"
    for f in sorted(src_dir.glob("*.cu")):
        for name, params in _DECL.findall(f.read_text()):
            letters = []
            plist = [q.strip() for q in params.split(",") if q.strip()]
            for q in plist:
                if "*" in q:
                    letters.append("p")
                elif q.startswith("unsigned long long"):
                    letters.append("u")
                elif q.startswith("long long"):
                    letters.append("l")
                elif q.startswith("float"):
                    letters.append("f")
                elif q.startswith("int"):
                    letters.append("i")
                else:
                    raise RuntimeError(f"unparsed parameter {q!r} in {name}")
            has_stream = bool(plist) and plist[-1].replace(" ", "") == "void*stream"
            sigs[name] = ("".join(letters[:-1]) if has_stream else "".join(letters), has_stream)
    return sigs


SIGS = _parse_sigs()

_CT = {"p": ctypes.c_void_p, "i": ctypes.c_int, "l": ctypes.c_longlong, "f": ctypes.c_float, "u": ctypes.c_ulonglong}


def lib_path() -> Path:
    return _LIB_PATH


def available() -> bool:
    return _LIB_PATH.exists()


def load():
    global _LIB
    if _LIB is not None:
        return _LIB
    if not _LIB_PATH.exists():
        raise RuntimeError(
            f"native kernel library not built: {_LIB_PATH} (run `python -m layerstorm_b200.build`)")
    lib = ctypes.CDLL(str(_LIB_PATH), mode=os.RTLD_GLOBAL if hasattr(os, "RTLD_GLOBAL") else ctypes.DEFAULT_MODE)
    for name, (sig, has_stream) in SIGS.items():
        fn = getattr(lib, name)
        fn.argtypes = [_CT[c] for c in sig] + ([ctypes.c_void_p] if has_stream else [])
        fn.restype = ctypes.c_int
    _LIB = lib
    return lib


_launches = 0
_timer = None          # list of (launcher, start event, end event) while a call_timer() is active


class call_timer:
    """``with call_timer() as t: ...`` brackets every launcher call made on the current stream with CUDA events (eager steps: the launchers'
    kernels run back to back, so a call's span is its kernels' device time plus the launch gap).  ``t.summary()`` -> {launcher: (calls, ms)}."""

    def __enter__(self):
        global _timer
        self.rec = []
        _timer = self.rec
        return self

    def __exit__(self, *exc):
        global _timer
        _timer = None
        return False

    def summary(self) -> dict:
        torch.cuda.synchronize()
        out = {}
        for name, e0, e1 in self.rec:
            c, ms = out.get(name, (0, 0.0))
            out[name] = (c + 1, ms + e0.elapsed_time(e1))
        return out


def launch_count() -> int:
    """Number of kernel-launcher calls made through :func:`call` in this process."""
    return _launches


def _ptr(x):
    if x is None:
        return None
    if isinstance(x, torch.Tensor):
        return x.data_ptr()
    return int(x)


def call(name: str, *args, stream=None):
    global _launches
    lib = load()
    sig, has_stream = SIGS[name]
    if len(args) != len(sig):
        raise TypeError(f"{name}: expected {len(sig)} args, got {len(args)}")
    conv = []
    for c, a in zip(sig, args):
        if c == "p":
            conv.append(_ptr(a))
        elif c == "f":
            conv.append(float(a))
        else:
            conv.append(int(a))
    if not has_stream:
        return getattr(lib, name)(*conv)
    st = stream if stream is not None else torch.cuda.current_stream().cuda_stream
    if _timer is not None:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        rc = getattr(lib, name)(*conv, st)
        e1.record()
        _timer.append((name, e0, e1))
    else:
        rc = getattr(lib, name)(*conv, st)
    _launches += 1
    if rc != 0:
        raise RuntimeError(f"{name} failed with status {rc}")
