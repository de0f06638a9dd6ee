"""The native host runtime under AddressSanitizer + UndefinedBehaviorSanitizer: the runtime's own tests (allocator, caches, tiers,
transfer engine, arena, rings, GGUF, ...) are re-run in a child process against a sanitized build of the library."""
import os
import shutil
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent


def test_native_runtime_tests_are_clean_under_asan_and_ubsan():
    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("no gcc")
    asan = subprocess.run([gcc, "-print-file-name=libasan.so"], capture_output=True, text=True).stdout.strip()
    if not os.path.isabs(asan) or not os.path.exists(asan):
        pytest.skip("the compiler ships no AddressSanitizer runtime")
    from layerstorm_b200 import build
    lib = build.build_sanitized("address,undefined")
    env = dict(os.environ, LD_PRELOAD=asan, ASAN_OPTIONS="detect_leaks=0:abort_on_error=0", UBSAN_OPTIONS="print_stacktrace=1",
               LSB200_RUNTIME_LIB=str(lib))
    files = ["test_runtime_native.py", "test_runtime_invariants.py", "test_runtime_tiers.py"]
    r = subprocess.run([sys.executable, "-m", "pytest", "-x", "-q", "-p", "no:cacheprovider"] + [str(ROOT / f) for f in files],
                       capture_output=True, text=True, env=env, timeout=900, cwd=str(ROOT.parent))
    out = r.stdout + r.stderr
    assert r.returncode == 0, out[-3000:]
    assert "AddressSanitizer" not in out and "runtime error:" not in out, out[-3000:]
    assert " passed" in r.stdout
