"""Expert-parallel routed-expert FFN with the exchange fused into the kernels.

``EpMoE.forward`` = dispatch (P2P stores of token rows into the expert owners' staging buffers) ->
tensor-core grouped gate/up+SwiGLU (prologue waits for the rows) -> tensor-core grouped down
(epilogue stores each output row into the token owner's buffer over NVLink) -> combine (waits, sums
the slots in order).  No collective library call on the path; NCCL / the process group is used only
to exchange buffer handles at construction.

``EpMoE.forward_nccl`` is the unfused baseline the fused path is measured against: the same grouped
GEMM kernels between two ``all_to_all_single`` exchanges.
Kernels: csrc/kernels/ep_moe.cu, csrc/kernels/moe_tc.cu.  Expert e is owned by rank e % world.
Reference call sites replaced: src/daemon/moe/moe_ranks.cpp:682-832 (EP broadcast + all-reduce).
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch
import torch.distributed as dist

from ..ops import _native as nat
from .symm import K_MAX_RANKS, SymmetricBuffer


class EpCommStruct(ctypes.Structure):
    _fields_ = [("nranks", ctypes.c_int), ("rank", ctypes.c_int), ("E", ctypes.c_int), ("_pad", ctypes.c_int),
                ("cap_rows", ctypes.c_longlong), ("max_pairs", ctypes.c_longlong), ("H", ctypes.c_int), ("_pad2", ctypes.c_int),
                ("cnt_all", ctypes.c_void_p * K_MAX_RANKS), ("xs", ctypes.c_void_p * K_MAX_RANKS), ("ret", ctypes.c_void_p * K_MAX_RANKS),
                ("y", ctypes.c_void_p * K_MAX_RANKS), ("flags", ctypes.c_void_p * K_MAX_RANKS),
                ("epoch", ctypes.c_void_p), ("cta_done", ctypes.c_void_p), ("err", ctypes.c_void_p)]


def _align(x: int, a: int = 256) -> int:
    return (x + a - 1) // a * a


class EpMoE:
    def __init__(self, hidden: int, inter: int, n_experts: int, top_k: int, max_tokens: int, device: torch.device, arena, group=None,
                 capacity_factor: float = 2.0, swiglu_limit: float = 0.0):
        """``arena``: ExpertArena holding this rank's experts (``slot_of[e] >= 0`` exactly for e % world == rank)."""
        self.group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(self.group), dist.get_world_size(self.group)
        assert self.world <= K_MAX_RANKS and hidden % 128 == 0 and inter % 128 == 0
        self.H, self.F, self.E, self.S = hidden, inter, n_experts, top_k
        self.dev, self.arena, self.limit = device, arena, swiglu_limit
        self.max_pairs = max_tokens * top_k
        # worst case every pair of every rank lands on one owner; capacity_factor x the average is the allocation
        self.cap_rows = min(self.world * self.max_pairs, int(capacity_factor * self.max_pairs) + 128 * n_experts // self.world)
        self.max_tiles = self.cap_rows // 32 + n_experts // self.world + 2      # sized for the smallest token tile
        sizes = {"cnt_all": self.world * n_experts * 4, "xs": self.cap_rows * hidden * 2, "ret": self.cap_rows * 8,
                 "y": self.max_pairs * hidden * 4, "flags": 3 * self.world * 4}
        offs, cur = {}, 0
        for k, v in sizes.items():
            offs[k] = cur
            cur += _align(v)
        self.symm = SymmetricBuffer(cur, device, self.group)
        i32 = dict(dtype=torch.int32, device=device)
        self.state = torch.zeros(16, **i32)                   # epoch | cta_done[4] | err
        self.dst_off, self.cursor = torch.zeros(n_experts, **i32), torch.zeros(n_experts, **i32)
        self.tile_e, self.tile_r0, self.tile_n = (torch.zeros(self.max_tiles, **i32) for _ in range(3))
        self.counters = torch.zeros(2, **i32)
        self.act = torch.zeros(self.cap_rows, inter, dtype=torch.float16, device=device)
        self.tc_err = torch.zeros(1, **i32)
        s = EpCommStruct()
        s.nranks, s.rank, s.E, s.cap_rows, s.max_pairs, s.H = self.world, self.rank, n_experts, self.cap_rows, self.max_pairs, hidden
        for p in range(self.world):
            b = self.symm.ptrs[p]
            s.cnt_all[p], s.xs[p], s.ret[p], s.y[p], s.flags[p] = (b + offs[k] for k in ("cnt_all", "xs", "ret", "y", "flags"))
        st = self.state.data_ptr()
        s.epoch, s.cta_done, s.err = st, st + 4, st + 20
        self.struct = s
        assert ctypes.sizeof(s) == nat.load().lsb_ep_comm_bytes(), "EpComm layout drifted from ep_comm.cuh"
        loc = self.symm.local
        self.xs_local = loc[offs["xs"]: offs["xs"] + sizes["xs"]].view(torch.float16).view(self.cap_rows, hidden)
        self.y_local = loc[offs["y"]: offs["y"] + sizes["y"]].view(torch.float32).view(self.max_pairs, hidden)
        self._base_ids = None

    @property
    def ptr(self) -> int:
        return ctypes.addressof(self.struct)

    def error(self) -> int:
        return int(self.state[5]) or int(self.tc_err)

    def rows_received(self) -> int:
        return int(self.counters[1])

    def _bn(self, R: int) -> int:
        """Token-tile width from the expected rows per owned expert (every rank must pick the same value)."""
        avg = R * self.S * self.world / self.E
        return 32 if avg <= 32 else (64 if avg <= 96 else 128)

    # ------------------------------------------------------------------ fused path
    def forward(self, x: torch.Tensor, ids: torch.Tensor, wts: torch.Tensor, out: torch.Tensor, accumulate: bool = False):
        """x bf16 [R, H]; ids int32 [R, S] (expert per slot, < 0 = none); wts fp32 [R, S]; out fp32 [R, H]."""
        R = x.shape[0]
        assert R * self.S <= self.max_pairs and ids.dtype == torch.int32 and x.dtype == torch.bfloat16
        efp = ctypes.addressof(self.arena.ef)
        self.BN = self._bn(R)
        nat.call("lsb_ep_dispatch", x, ids, R * self.S, self.S, self.BN, self.dst_off, self.cursor, self.tile_e, self.tile_r0, self.tile_n,
                 self.counters, self.max_tiles, self.ptr)
        for gateup, b, o, lim in ((1, self.xs_local, self.act, self.limit), (0, self.act, self.y_local, 0.0)):
            nat.call("lsb_moe_tc_ffn", gateup, b, self.cap_rows, self.arena.data, self.arena.slot_of, efp, self.tile_e, self.tile_r0, self.tile_n,
                     self.counters, None, o, self.BN, self.max_tiles, lim, None, self.tc_err, self.ptr)
        nat.call("lsb_ep_combine", out, wts, ids, R, self.S, int(accumulate), self.ptr)
        return out

    # ------------------------------------------------------------------ unfused baseline
    def _nccl_buffers(self):
        if getattr(self, "_nb", None) is None:
            dev, i32 = self.dev, dict(dtype=torch.int32, device=self.dev)
            tiles = self.cap_rows // 32 + self.E + 2
            self._nb = dict(srt=torch.zeros(self.cap_rows, **i32), te=torch.zeros(tiles, **i32), tr=torch.zeros(tiles, **i32),
                            tn=torch.zeros(tiles, **i32), cnt=torch.zeros(2, **i32), xs=torch.zeros(self.cap_rows, self.H, dtype=torch.float16, device=dev),
                            y=torch.zeros(self.cap_rows, self.H, device=dev), tiles=tiles)
        return self._nb

    def forward_nccl(self, x: torch.Tensor, ids: torch.Tensor, wts: torch.Tensor, out: torch.Tensor):
        """The library baseline WITHOUT a host round trip: fixed-capacity all-to-all.  Every rank sends every peer a slab of
        ``cap = cap_rows / world`` rows (its pairs for that peer's experts in expert order, the rest padding with expert id -1), so
        the split sizes are constants and nothing has to come back to the host before the exchange; the grouped GEMMs run over the
        received slabs (padding rows are ignored by the tile builder), the results travel back slab by slab.  Same GEMM kernels as
        ``forward``.  Pairs beyond a slab's capacity would be dropped (``cap_rows`` is sized with the capacity factor of the fused
        path; the test checks equality, i.e. that nothing was dropped)."""
        W, S, H = self.world, self.S, self.H
        R = x.shape[0]
        P = R * S
        cap = self.cap_rows // W
        dev = x.device
        flat = ids.reshape(-1).long()
        owner = flat % W
        order = torch.argsort(owner * self.E + flat, stable=True)                # by owner, then expert
        so = owner[order]
        counts = torch.bincount(owner, minlength=W)
        starts = torch.cumsum(counts, 0) - counts
        rank_in = torch.arange(P, device=dev) - starts[so]
        slot = torch.where(rank_in < cap, so * cap + rank_in, torch.full_like(so, W * cap))     # overflow -> the dump row
        send_x = torch.zeros(W * cap + 1, H, dtype=x.dtype, device=dev)
        send_e = torch.full((W * cap + 1,), -1, dtype=torch.int32, device=dev)
        send_x.index_copy_(0, slot, x[order // S])
        send_e.index_copy_(0, slot, flat[order].int())
        recv_x = torch.empty(W * cap, H, dtype=x.dtype, device=dev)
        recv_e = torch.empty(W * cap, dtype=torch.int32, device=dev)
        dist.all_to_all_single(recv_x, send_x[: W * cap], group=self.group)
        dist.all_to_all_single(recv_e, send_e[: W * cap], group=self.group)
        nb = self._nccl_buffers()
        efp = ctypes.addressof(self.arena.ef)
        self.BN = self._bn(R)
        n_recv = W * cap
        nat.call("lsb_moe_tc_sort", recv_e, n_recv, self.E, self.BN, nb["srt"], nb["te"], nb["tr"], nb["tn"], nb["cnt"])
        nat.call("lsb_moe_tc_gather", recv_x, nb["srt"], nb["cnt"], nb["xs"], n_recv, 1, H)
        nat.call("lsb_moe_tc_ffn", 1, nb["xs"], self.cap_rows, self.arena.data, self.arena.slot_of, efp, nb["te"], nb["tr"], nb["tn"], nb["cnt"],
                 nb["srt"], self.act, self.BN, nb["tiles"], self.limit, None, self.tc_err, None)
        nat.call("lsb_moe_tc_ffn", 0, self.act, self.cap_rows, self.arena.data, self.arena.slot_of, efp, nb["te"], nb["tr"], nb["tn"], nb["cnt"],
                 nb["srt"], nb["y"], self.BN, nb["tiles"], 0.0, None, self.tc_err, None)
        back = torch.empty(W * cap + 1, H, device=dev)
        dist.all_to_all_single(back[: W * cap], nb["y"][: W * cap], group=self.group)
        back[W * cap].zero_()
        y = torch.empty(P, H, device=dev)
        y[order] = back[slot]
        out.copy_((y.view(R, S, H) * wts.unsqueeze(-1)).sum(1))
        return out

    def forward_nccl_variable(self, x: torch.Tensor, ids: torch.Tensor, wts: torch.Tensor, out: torch.Tensor):
        """all_to_all(tokens) with exact split sizes -> grouped GEMMs -> all_to_all(results) -> weighted sum.  The split sizes have to
        reach the host first (one ``.tolist()`` round trip per call); kept as the second baseline."""
        W, S, H = self.world, self.S, self.H
        R = x.shape[0]
        flat = ids.reshape(-1).long()
        owner = flat % W
        order = torch.argsort(owner * self.E + flat, stable=True)                # by owner, then expert
        send_counts = torch.bincount(owner, minlength=W)
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts, group=self.group)
        sc, rc = send_counts.tolist(), recv_counts.tolist()                        # host sync: the library needs split sizes
        n_recv = sum(rc)
        assert n_recv <= self.cap_rows
        send_x = x[order // S].contiguous()
        send_e = flat[order].int()
        recv_x = torch.empty(n_recv, H, dtype=x.dtype, device=x.device)
        recv_e = torch.empty(n_recv, dtype=torch.int32, device=x.device)
        dist.all_to_all_single(recv_x, send_x, rc, sc, group=self.group)
        dist.all_to_all_single(recv_e, send_e, rc, sc, group=self.group)
        nb = self._nccl_buffers()
        efp = ctypes.addressof(self.arena.ef)
        self.BN = self._bn(R)
        if n_recv:
            nat.call("lsb_moe_tc_sort", recv_e, n_recv, self.E, self.BN, nb["srt"], nb["te"], nb["tr"], nb["tn"], nb["cnt"])
            nat.call("lsb_moe_tc_gather", recv_x, nb["srt"], nb["cnt"], nb["xs"], n_recv, 1, H)
            nat.call("lsb_moe_tc_ffn", 1, nb["xs"], self.cap_rows, self.arena.data, self.arena.slot_of, efp, nb["te"], nb["tr"], nb["tn"], nb["cnt"],
                     nb["srt"], self.act, self.BN, nb["tiles"], self.limit, None, self.tc_err, None)
            nat.call("lsb_moe_tc_ffn", 0, self.act, self.cap_rows, self.arena.data, self.arena.slot_of, efp, nb["te"], nb["tr"], nb["tn"], nb["cnt"],
                     nb["srt"], nb["y"], self.BN, nb["tiles"], 0.0, None, self.tc_err, None)
        back = torch.empty(R * S, H, device=x.device)
        dist.all_to_all_single(back, nb["y"][:n_recv], sc, rc, group=self.group)
        y = torch.empty_like(back)
        y[order] = back
        out.copy_((y.view(R, S, H) * wts.unsqueeze(-1)).sum(1))
        return out


def zipf_router(tokens: int, n_experts: int, top_k: int, device, seed: int = 0, alpha: float = 1.1):
    """Routing of the expert-parallel microbenchmark: logits N(0,1) plus a Zipf(alpha) per-expert bias; softmax
    weights over the selected experts."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    ranks = torch.arange(1, n_experts + 1, dtype=torch.float32)
    bias = torch.log(ranks.pow(-alpha) / ranks.pow(-alpha).sum())
    bias = bias[torch.randperm(n_experts, generator=g)]
    logits = torch.randn(tokens, n_experts, generator=g) + bias
    val, idx = torch.topk(logits, top_k, dim=-1)
    return idx.int().to(device).contiguous(), torch.softmax(val, -1).to(device).contiguous()
