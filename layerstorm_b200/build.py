"""In-tree native build: compiles every CUDA kernel file for sm_100a and every C++
runtime file into shared libraries under ``layerstorm_b200/_lib``.

Two libraries are produced:

* ``liblsb200_kernels.so``  - all ``csrc/kernels/*.cu`` (device code, sm_100a only)
* ``liblsb200_runtime.so``  - all ``csrc/runtime/*.cpp`` (host-only C++20 runtime)

The libraries expose a plain C ABI and are loaded with ``ctypes`` (see
``layerstorm_b200/ops/_native.py`` and ``layerstorm_b200/runtime/_native.py``), so no
Python headers are needed and a full rebuild takes well under a minute.  Objects are
cached by a content hash of the source, the shared headers and the flags.
"""
from __future__ import annotations

import concurrent.futures as cf
import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
LIB = ROOT / "_lib"
OBJ = LIB / "obj"

NVCC = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
CXX = os.environ.get("CXX") or shutil.which("g++") or "g++"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=default",
    "-I", str(CSRC / "include"), "-I", str(CSRC / "kernels"),
]
CXX_FLAGS = ["-O2", "-g", "-std=c++20", "-fPIC", "-Wall", "-Wno-unused-function", "-pthread",
             "-I", str(CSRC / "include"), "-I", str(CSRC / "runtime")]


def _hash(paths, flags) -> str:
    h = hashlib.sha256()
    for p in paths:
        h.update(str(p).encode())
        h.update(Path(p).read_bytes())
    h.update(" ".join(flags).encode())
    return h.hexdigest()[:16]


def _headers():
    hs = sorted(CSRC.rglob("*.h")) + sorted(CSRC.rglob("*.cuh")) + sorted(CSRC.rglob("*.hpp"))
    return hs


def _compile_one(src: Path, kind: str, verbose: bool) -> Path:
    flags = NVCC_FLAGS if kind == "cu" else CXX_FLAGS
    key = _hash([src] + _headers(), flags)
    obj = OBJ / f"{src.stem}.{key}.o"
    if obj.exists():
        return obj
    for old in OBJ.glob(f"{src.stem}.*.o"):
        old.unlink()
    if kind == "cu":
        cmd = [NVCC] + flags + (["-Xptxas", "-v"] if verbose else []) + ["-c", str(src), "-o", str(obj)]
    else:
        cmd = [CXX] + flags + ["-c", str(src), "-o", str(obj)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"compile failed: {' '.join(cmd)}\n{r.stdout}\n{r.stderr}")
    if verbose:
        sys.stderr.write(r.stderr)
    return obj


def _link(objs, out: Path, kind: str):
    stamp = out.with_suffix(".stamp")
    key = hashlib.sha256(" ".join(sorted(str(o) for o in objs)).encode()).hexdigest()
    if out.exists() and stamp.exists() and stamp.read_text() == key:
        return
    if kind == "cu":
        cmd = [NVCC, "-shared", "-o", str(out)] + [str(o) for o in objs] + []
    else:
        cmd = [CXX, "-shared", "-o", str(out)] + [str(o) for o in objs] + ["-pthread", "-ldl", "-lrt"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed: {' '.join(cmd)}\n{r.stdout}\n{r.stderr}")
    stamp.write_text(key)


def build_all(verbose: bool = False, only: str | None = None) -> dict:
    """Build both libraries; returns {name: path}."""
    OBJ.mkdir(parents=True, exist_ok=True)
    out = {}
    jobs = []
    cu = sorted((CSRC / "kernels").glob("*.cu"))
    cpp = sorted((CSRC / "runtime").glob("*.cpp"))
    with cf.ThreadPoolExecutor(max_workers=max(2, (os.cpu_count() or 4))) as ex:
        if only in (None, "kernels"):
            jobs += [("cu", ex.submit(_compile_one, s, "cu", verbose)) for s in cu]
        if only in (None, "runtime"):
            jobs += [("cpp", ex.submit(_compile_one, s, "cpp", verbose)) for s in cpp]
        objs = {"cu": [], "cpp": []}
        for kind, fut in jobs:
            objs[kind].append(fut.result())
    if objs["cu"]:
        p = LIB / "liblsb200_kernels.so"
        _link(objs["cu"], p, "cu")
        out["kernels"] = p
    if objs["cpp"]:
        p = LIB / "liblsb200_runtime.so"
        _link(objs["cpp"], p, "cpp")
        out["runtime"] = p
    return out


def build_sanitized(sanitizers: str = "address,undefined") -> Path:
    """The host runtime built with -fsanitize=<sanitizers> into ``_lib/liblsb200_runtime_san.so`` (the production library is not touched).
    Load it with ``LSB200_RUNTIME_LIB=<path>`` and the sanitizer runtime preloaded (``LD_PRELOAD=$(gcc -print-file-name=libasan.so)``):
    ``tests/test_runtime_sanitized.py`` runs the native-runtime tests that way.  The kernels library has no sanitized build
    (compute-sanitizer is the tool for device code)."""
    obj = OBJ / ("san_" + sanitizers.replace(",", "_"))
    obj.mkdir(parents=True, exist_ok=True)
    cxx = os.environ.get("LSB200_SAN_CXX") or shutil.which("g++") or CXX        # the distribution's compiler ships the sanitizer runtimes
    flags = [f for f in CXX_FLAGS if not f.startswith("-O")] + ["-O1", "-g", "-fno-omit-frame-pointer", f"-fsanitize={sanitizers}"]
    objs = []
    for src in sorted((CSRC / "runtime").glob("*.cpp")):
        o = obj / f"{src.stem}.{_hash([src] + _headers(), flags)}.o"
        if not o.exists():
            for old in obj.glob(f"{src.stem}.*.o"):
                old.unlink()
            r = subprocess.run([cxx] + flags + ["-c", str(src), "-o", str(o)], capture_output=True, text=True)
            if r.returncode != 0:
                raise RuntimeError(f"compile failed: {src}\n{r.stderr}")
        objs.append(o)
    out = LIB / "liblsb200_runtime_san.so"
    r = subprocess.run([cxx, "-shared", f"-fsanitize={sanitizers}", "-o", str(out)] + [str(o) for o in objs] + ["-pthread", "-ldl", "-lrt"],
                       capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed\n{r.stderr}")
    return out


if __name__ == "__main__":
    if "--sanitize" in sys.argv:
        print("runtime (sanitized)", build_sanitized(sys.argv[sys.argv.index("--sanitize") + 1] if len(sys.argv) > sys.argv.index("--sanitize") + 1 else "address,undefined"))
        sys.exit(0)
    res = build_all(verbose="-v" in sys.argv)
    for k, v in res.items():
        print(k, v)
