"""ThreadSanitizer over the host-runtime components shared between two threads (SPSC ring, seqlock snapshot, NVMe tier worker pool, host arena with concurrent loaders, CPU expert fork-join pool):
a small C++ driver is built with -fsanitize=thread from the runtime sources and run; any TSAN report fails it."""
import shutil
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent
RUNTIME = ROOT.parent / "layerstorm_b200" / "csrc" / "runtime"


def test_shared_runtime_components_are_race_free(tmp_path):
    gxx = shutil.which("g++")
    if gxx is None:
        pytest.skip("no g++")
    tsan = subprocess.run([gxx, "-print-file-name=libtsan.so"], capture_output=True, text=True).stdout.strip()
    if "/" not in tsan:
        pytest.skip("the compiler ships no ThreadSanitizer runtime")
    exe = tmp_path / "tsan_driver"
    r = subprocess.run([gxx, "-O1", "-g", "-std=c++20", "-fsanitize=thread", "-pthread", "-w", "-I", str(RUNTIME.parent / "include"), "-I", str(RUNTIME),
                        str(ROOT / "native" / "tsan_driver.cpp"), str(RUNTIME / "ipc.cpp"), str(RUNTIME / "nvme_tier.cpp"), str(RUNTIME / "host_arena.cpp"), str(RUNTIME / "cpu_experts.cpp"), str(RUNTIME / "gguf.cpp"), "-o", str(exe)],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-2000:]
    store = tmp_path / "nvme"
    store.mkdir()
    r = subprocess.run([str(exe), str(store)], capture_output=True, text=True, timeout=600)
    out = r.stdout + r.stderr
    assert r.returncode == 0 and "TSAN_DRIVER_OK" in out, out[-3000:]
    assert "ThreadSanitizer" not in out, out[-3000:]
