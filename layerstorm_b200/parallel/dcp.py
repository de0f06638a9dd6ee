"""Context-parallel ("DCP", sharded KV) absorbed-MLA attention.

The latent KV cache is sharded by token position over the ranks (round-robin in chunks of ``chunk`` tokens, each rank
keeps its tokens compacted in its local paged cache); the query heads stay tensor-parallel.  ``DcpAttention.forward``
= all-gather of the absorbed queries in the head dimension (P2P stores) -> split-KV attention of ALL heads over the
local token shard (the ordinary ``lsb_mla_decode`` kernels, partials only) -> partials stored straight into the head
owners' buffers -> log-sum-exp merge on the head owner.  No collective library call on the path; NCCL / the process
group only exchanges buffer handles at construction.  Kernels: csrc/kernels/dcp.cu.
Reference behaviour replaced: ``hardware.dcp_kv_mode = sharded`` (all-gather Q, all-gather LSE, lse-correct, all-reduce
of [B, H, D_c], slice; src/daemon/attention/arch_mla.cpp:2555-2574, src/parallelism/dcp_communicator.cpp).
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch
import torch.distributed as dist

from ..ops import _native as nat
from .symm import K_MAX_RANKS, SymmetricBuffer


class DcpCommStruct(ctypes.Structure):
    _fields_ = [("nranks", ctypes.c_int), ("rank", ctypes.c_int), ("H", ctypes.c_int), ("Hh", ctypes.c_int),
                ("D", ctypes.c_int), ("dl", ctypes.c_int), ("NS", ctypes.c_int), ("max_rows", ctypes.c_int),
                ("q_all", ctypes.c_void_p * K_MAX_RANKS), ("part", ctypes.c_void_p * K_MAX_RANKS), ("flags", ctypes.c_void_p * K_MAX_RANKS),
                ("epoch", ctypes.c_void_p), ("cta_done", ctypes.c_void_p), ("err", ctypes.c_void_p)]


def _align(x: int, a: int = 256) -> int:
    return (x + a - 1) // a * a


def owner_of(pos: int, chunk: int, world: int) -> int:
    """Rank that stores token position ``pos``."""
    return (pos // chunk) % world


def local_index(pos: int, chunk: int, world: int) -> int:
    """Index of an owned position inside its rank's compacted shard."""
    return (pos // (chunk * world)) * chunk + pos % chunk


def local_length(length: int, chunk: int, world: int, rank: int) -> int:
    """How many of the positions [0, length) rank ``rank`` stores."""
    full, rem = divmod(length, chunk * world)
    return full * chunk + min(max(rem - rank * chunk, 0), chunk)


class DcpAttention:
    def __init__(self, n_heads: int, dl: int, dr: int, max_rows: int, device: torch.device, group=None, chunk: int = 64, n_splits: int = 4):
        self.group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(self.group), dist.get_world_size(self.group)
        assert self.world <= K_MAX_RANKS and n_heads % self.world == 0
        self.H, self.Hh, self.dl, self.dr, self.D = n_heads, n_heads // self.world, dl, dr, dl + dr
        self.max_rows, self.NS, self.chunk, self.dev = max_rows, n_splits, chunk, device
        sizes = {"q_all": max_rows * self.H * self.D * 2, "part": self.world * max_rows * self.Hh * self.NS * (dl + 4) * 4,
                 "flags": 2 * self.world * 4}
        offs, cur = {}, 0
        for k, v in sizes.items():
            offs[k] = cur
            cur += _align(v)
        self.symm = SymmetricBuffer(cur, device, self.group)
        self.state = torch.zeros(8, dtype=torch.int32, device=device)            # epoch | cta_done[2] | err
        s = DcpCommStruct()
        s.nranks, s.rank, s.H, s.Hh, s.D, s.dl, s.NS, s.max_rows = self.world, self.rank, self.H, self.Hh, self.D, dl, self.NS, max_rows
        for p in range(self.world):
            b = self.symm.ptrs[p]
            s.q_all[p], s.part[p], s.flags[p] = (b + offs[k] for k in ("q_all", "part", "flags"))
        st = self.state.data_ptr()
        s.epoch, s.cta_done, s.err = st, st + 4, st + 12
        self.struct = s
        assert ctypes.sizeof(s) == nat.load().lsb_dcp_comm_bytes(), "DcpComm layout drifted from dcp.cu"
        loc = self.symm.local
        self.q_all = loc[offs["q_all"]: offs["q_all"] + sizes["q_all"]].view(torch.bfloat16).view(max_rows, self.H, self.D)
        self.o_part = torch.zeros(max_rows, self.H, self.NS, dl, device=device)
        self.ml_part = torch.zeros(max_rows, self.H, self.NS, 2, device=device)
        self.loc_idx: Optional[torch.Tensor] = None
        self.loc_cnt = torch.zeros(max_rows, dtype=torch.int32, device=device)

    @property
    def ptr(self) -> int:
        return ctypes.addressof(self.struct)

    def error(self) -> int:
        return int(self.state[3])

    def error_word(self) -> torch.Tensor:
        """One-element view of the kernels' error word (read back by the engine with every step's tokens)."""
        return self.state[3:4]

    def forward(self, q_local: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor, max_pages: int, row_seq: torch.Tensor,
                row_len_local: torch.Tensor, out: torch.Tensor, page: int, kv_fmt: int, scale: float, sel_idx: Optional[torch.Tensor] = None,
                sel_cnt: Optional[torch.Tensor] = None, tq_centroids: Optional[torch.Tensor] = None, lse: Optional[torch.Tensor] = None,
                rows: Optional[int] = None):
        """q_local bf16 [R, Hh, D] (this rank's heads); cache / block_table: this rank's token shard; row_len_local int32 [R]:
        owned positions visible to each row (``local_length``); sel_idx / sel_cnt: the indexer's GLOBAL positions (sparse
        layers) or None; out bf16 [R, Hh, dl]."""
        R = rows if rows is not None else q_local.shape[0]          # `rows`: only the first rows of a larger static buffer are live
        assert R <= self.max_rows and q_local.dtype == torch.bfloat16 and q_local.is_contiguous()
        nat.call("lsb_dcp_gather_q", q_local, R, self.ptr)
        li = lc = None
        sel_ld = 0
        if sel_idx is not None:
            sel_ld = sel_idx.shape[1]
            if self.loc_idx is None or self.loc_idx.shape[1] != sel_ld:
                self.loc_idx = torch.zeros(self.max_rows, sel_ld, dtype=torch.int32, device=self.dev)
            li, lc = self.loc_idx, self.loc_cnt
            nat.call("lsb_dcp_localize", sel_idx, sel_cnt, sel_ld, li, lc, R, self.chunk, self.world, self.rank)
        nat.call("lsb_mla_decode", self.q_all, cache, block_table, max_pages, row_seq, row_len_local, li, lc, sel_ld, None, None,
                 self.o_part, self.ml_part, R, self.H, self.dl, self.dr, page, kv_fmt, self.NS, scale, tq_centroids)
        nat.call("lsb_dcp_scatter_combine", self.o_part, self.ml_part, out, lse, R, self.ptr)
        return out
