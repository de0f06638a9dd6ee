"""The allocation-free argmax entry point, called through its exported C symbol.

Callers that may not allocate device memory (a frozen memory pool, an embedding application that
owns the device heap) use ``lsb_argmax_noalloc``; it must give exactly what the regular entry
point gives, call after call, because its internal scratch array is reused between calls.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

from layerstorm_b200.ops import _native as nat


def test_noalloc_argmax_matches_regular_entry_point_twice():
    lib = ctypes.CDLL(str(nat.lib_path()))
    fn = lib.lsb_argmax_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p]
    lib.lsb_argmax_noalloc_max_rows.restype = ctypes.c_int
    max_rows = lib.lsb_argmax_noalloc_max_rows()
    assert max_rows == 256
    st = torch.cuda.current_stream().cuda_stream
    for call, (rows, V) in enumerate([(7, 50021), (3, 1031), (max_rows, 257)]):     # the last case touches the whole fixed array
        g = torch.Generator().manual_seed(100 + call)
        logits = (torch.randn(rows, V, generator=g) * 3).cuda()
        logits[0, 5] = logits[0, V - 2] = 99.0                 # tie: the lower index must win
        part = torch.zeros(rows, 64, dtype=torch.int64, device="cuda")
        ref_ids = torch.zeros(rows, dtype=torch.int32, device="cuda")
        ref_val = torch.zeros(rows, device="cuda")
        nat.call("lsb_argmax", logits, V, rows, V, part, ref_ids, ref_val, 11, None)
        ids = torch.full((rows,), -1, dtype=torch.int32, device="cuda")
        val = torch.zeros(rows, device="cuda")
        rc = fn(logits.data_ptr(), V, rows, V, ids.data_ptr(), val.data_ptr(), 11, st)
        assert rc == 0
        torch.cuda.synchronize()
        assert torch.equal(ids, ref_ids) and torch.equal(val, ref_val)
        assert int(ids[0]) == 11 + 5
        assert torch.equal(ids[1:].cpu().long() - 11, logits[1:].cpu().argmax(-1))
    # a row stride shorter than the row is refused
    assert fn(logits.data_ptr(), V - 1, rows, V, ids.data_ptr(), None, 0, st) == -1
    # beyond the fixed scratch size the call is refused and nothing runs
    big = torch.zeros(max_rows + 1, 8, device="cuda")
    out = torch.full((max_rows + 1,), -7, dtype=torch.int32, device="cuda")
    assert fn(big.data_ptr(), 8, max_rows + 1, 8, out.data_ptr(), None, 0, st) == -2
    torch.cuda.synchronize()
    assert int(out[0]) == -7
