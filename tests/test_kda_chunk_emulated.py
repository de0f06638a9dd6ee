"""The CUDA source of the chunk-parallel KDA kernels, executed on the CPU by a SIMT emulation (one OS thread per CUDA thread, barriers
for __syncthreads, buffer exchange for warp shuffles), against the token-by-token recurrence.  Covers full and partial chunks, a row
offset, a non-zero state slot, the conv-history update and the untouched neighbour slot."""
import shutil
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent
KERNELS = ROOT.parent / "layerstorm_b200" / "csrc" / "kernels"


@pytest.fixture(scope="module")
def emulator(tmp_path_factory):
    gxx = shutil.which("g++")
    if gxx is None:
        pytest.skip("no g++")
    exe = tmp_path_factory.mktemp("emu") / "kda_chunk_emu"
    r = subprocess.run([gxx, "-O1", "-std=c++20", "-pthread", "-w", "-I", str(KERNELS), str(ROOT / "simt_emu" / "kda_chunk_emu.cpp"), "-o", str(exe)],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-2000:]
    return exe


@pytest.mark.parametrize("tokens,heads", [(150, 2), (128, 1), (65, 1)])
def test_chunk_kernels_match_the_recurrence(emulator, tokens, heads):
    r = subprocess.run([str(emulator), str(tokens), str(heads)], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "conv_ok=1" in r.stdout and "other_slot_untouched=1" in r.stdout
