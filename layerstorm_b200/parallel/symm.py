"""Peer-mapped symmetric buffers for the in-kernel NVLink collectives.

One process per GPU (torchrun).  Every rank allocates the same buffers; the device
pointers of all ranks' copies are exchanged so kernels can store straight into peer memory
over NVLink / NVSwitch.  ``torch.distributed._symmetric_memory`` does the allocation and
handle exchange when available; otherwise CUDA IPC handles are exchanged through the
process group.  NCCL is used only for this bootstrap, never on the per-layer path.

The resulting ``PeerComm`` ctypes struct mirrors ``lsb::PeerComm`` (csrc/kernels/comm.cuh)
and is passed by value into the producer / consumer kernels.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional

import torch
import torch.distributed as dist

K_MAX_RANKS = 8
LL_ELEMS = 65536     # elements per slot of the flag-in-data exchange buffers (8 rows of hidden 8192), see PeerComm


class PeerCommStruct(ctypes.Structure):
    _fields_ = [("nranks", ctypes.c_int), ("rank", ctypes.c_int), ("cap", ctypes.c_longlong),
                ("recv", ctypes.c_void_p * K_MAX_RANKS), ("flags", ctypes.c_void_p * K_MAX_RANKS),
                ("epoch", ctypes.c_void_p), ("cta_done", ctypes.c_void_p), ("err", ctypes.c_void_p), ("xchg", ctypes.c_int),
                ("ll_cap", ctypes.c_longlong), ("ll", ctypes.c_void_p * K_MAX_RANKS)]


class SymmetricBuffer:
    """A byte buffer allocated on every rank with all peers' device pointers known."""

    def __init__(self, nbytes: int, device: torch.device, group=None):
        self.group = group if group is not None else dist.group.WORLD
        self.rank = dist.get_rank(self.group)
        self.world = dist.get_world_size(self.group)
        self.nbytes = nbytes
        self.ptrs: List[int] = []
        self._keep = []
        self.backend = None
        try:
            import torch.distributed._symmetric_memory as symm_mem
            t = symm_mem.empty(nbytes, dtype=torch.uint8, device=device)
            hdl = symm_mem.rendezvous(t, group=self.group)
            self.local = t
            self.ptrs = [int(p) for p in hdl.buffer_ptrs]
            self._keep.append(hdl)
            self.backend = "symmetric_memory"
        except Exception as exc:  # noqa: BLE001 - fall back to raw CUDA IPC
            self._ipc_fallback(nbytes, device, exc)
        self.local.zero_()
        torch.cuda.synchronize(device)
        dist.barrier(self.group)

    def _ipc_fallback(self, nbytes: int, device: torch.device, why: Exception):
        t = torch.zeros(nbytes, dtype=torch.uint8, device=device)
        handle = t.untyped_storage()._share_cuda_()
        handles = [None] * self.world
        dist.all_gather_object(handles, handle, group=self.group)
        self.local = t
        for r, h in enumerate(handles):
            if r == self.rank:
                self.ptrs.append(t.data_ptr())
                continue
            st = torch.UntypedStorage._new_shared_cuda(*h)
            peer = torch.empty(0, dtype=torch.uint8, device=st.device).set_(st)
            self._keep.append(peer)
            self.ptrs.append(peer.data_ptr())
        self.backend = f"cuda_ipc (symmetric_memory unavailable: {type(why).__name__})"


class PeerComm:
    """Receive slots + flags for the fused all-reduce (see csrc/kernels/comm.cuh)."""

    def __init__(self, cap_floats: int, device: torch.device, group=None):
        group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        assert self.world <= K_MAX_RANKS
        cap_floats = (cap_floats + 3) // 4 * 4
        self.cap = cap_floats
        recv_bytes = 2 * self.world * cap_floats * 4
        # producer-push flags [2][8] + consumer-exchange flags [2][8 ranks][128 CTAs] (see csrc/kernels/comm.cuh)
        flag_bytes = (2 * K_MAX_RANKS + 2 * K_MAX_RANKS * 128) * 4
        # flag-in-data buffers of the few-row exchange: [2 parities][ranks][ll_cap] words of (value, epoch), 8 bytes each
        self.ll_cap = (min(cap_floats, LL_ELEMS) + 3) // 4 * 4
        ll_bytes = 2 * self.world * self.ll_cap * 8
        self.buf = SymmetricBuffer(recv_bytes + flag_bytes + ll_bytes, device, group)
        self.local_state = torch.zeros(16, dtype=torch.int32, device=device)   # epoch, cta_done, err
        s = PeerCommStruct()
        s.nranks, s.rank, s.cap = self.world, self.rank, cap_floats
        for p in range(self.world):
            s.recv[p] = self.buf.ptrs[p]
            s.flags[p] = self.buf.ptrs[p] + recv_bytes
            s.ll[p] = self.buf.ptrs[p] + recv_bytes + flag_bytes
        base = self.local_state.data_ptr()
        s.epoch, s.cta_done, s.err = base, base + 4, base + 8
        s.xchg = 0
        s.ll_cap = self.ll_cap
        self.struct = s

    @property
    def ptr(self) -> int:
        return ctypes.addressof(self.struct)

    def error(self) -> int:
        return int(self.local_state[2])

    def epoch(self) -> int:
        return int(self.local_state[0])
