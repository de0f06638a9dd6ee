"""Device-resident model: weights in the kernels' storage formats plus the per-step forward
pass expressed as a fixed sequence of hand-written kernel launches (CUDA-graph capturable:
all shapes are static for a given workspace, all data-dependent quantities live on the
device).

Weight formats: bf16, FP8 e4m3 with 128x128 block scales, NVFP4 (16-wide e4m3 scales in the
128x4 atom layout + per-tensor scale).  Routed and shared experts live in a slotted arena
per MoE layer (``slot_of[expert] -> slot`` or -1), which is what the VRAM expert cache
manipulates.  Reference structure: LoadedModel / LayerWeights (src/model/weight_loader),
the per-layer bodies src/daemon/attention/arch_mla.cpp, arch_glm5_next.cpp and
src/daemon/moe/moe_driver.cpp:382-1745.
"""
from __future__ import annotations

import os

import ctypes
import math
from dataclasses import dataclass
from typing import Dict, List, Optional

import torch

from ..formats import quant
from ..ops import _native as nat
from .config import ModelConfig

KV_FMT = {"bf16": 0, "fp8": 1, "tq4": 2}
EXPERT_FMT = {"bf16": 0, "fp8_e4m3": 1, "nvfp4": 2, "gguf_q4_k": 3, "gguf_q5_k": 4, "gguf_q6_k": 5, "gguf_q8_0": 6}
_FMT_NAME = {v: k for k, v in EXPERT_FMT.items()}
GGML_OF = {"gguf_q4_k": 12, "gguf_q5_k": 13, "gguf_q6_k": 14, "gguf_q8_0": 8}      # storage formats that are GGUF block types


class ExpertFmt(ctypes.Structure):
    _fields_ = [("fmt", ctypes.c_int), ("H", ctypes.c_int), ("F", ctypes.c_int),
                ("stride", ctypes.c_longlong),
                ("off_gate", ctypes.c_longlong), ("off_up", ctypes.c_longlong), ("off_down", ctypes.c_longlong),
                ("off_sg", ctypes.c_longlong), ("off_su", ctypes.c_longlong), ("off_sd", ctypes.c_longlong),
                ("off_tail", ctypes.c_longlong), ("fmt_down1", ctypes.c_int)]


def _align(x, a):
    return (x + a - 1) // a * a


def expert_layout(fmt: str, H: int, F: int, down_fmt: Optional[str] = None) -> ExpertFmt:
    """Byte layout of one expert slot (gate | up | down weights, then their scales, then a tail
    of per-tensor scales), slot stride 4096-aligned like the reference's prepacked slots
    (src/model/weight_pipeline/prepacked_format.h:44-52).  ``down_fmt``: GGUF files mix block types per tensor; the down
    matrix may be another GGUF block type than gate / up."""
    ef = ExpertFmt()
    ef.fmt, ef.H, ef.F = EXPERT_FMT[fmt], H, F
    if fmt in GGML_OF and (fmt != "gguf_q4_k" or (down_fmt or fmt) != fmt):
        from ..formats import gguf as _gguf
        dfmt = down_fmt or fmt
        if dfmt not in GGML_OF or H % 256 or F % 256:
            raise ValueError("GGUF block-type experts need hidden and intermediate sizes that are multiples of 256 and a GGUF block type for the down matrix")
        gu = _align(F * _gguf.device_row_bytes(GGML_OF[fmt], H), 256)
        dn = _align(H * _gguf.device_row_bytes(GGML_OF[dfmt], F), 256)
        ef.off_gate, ef.off_up, ef.off_down = 0, gu, 2 * gu
        ef.off_sg = ef.off_su = ef.off_sd = ef.off_tail = 2 * gu + dn
        ef.fmt_down1 = 0 if dfmt == fmt else EXPERT_FMT[dfmt] + 1
        ef.stride = _align(2 * gu + dn, 4096)
        return ef
    if down_fmt not in (None, fmt):
        raise ValueError("a separate down format is only supported between GGUF block types")
    if fmt == "bf16":
        wb = H * F * 2
        ef.off_gate, ef.off_up, ef.off_down = 0, wb, 2 * wb
        ef.off_sg = ef.off_su = ef.off_sd = ef.off_tail = 3 * wb
        end = 3 * wb
    elif fmt == "fp8_e4m3":
        wb = H * F
        ef.off_gate, ef.off_up, ef.off_down = 0, wb, 2 * wb
        sgu = ((F + 127) // 128) * ((H + 127) // 128) * 4
        sd = ((H + 127) // 128) * ((F + 127) // 128) * 4
        ef.off_sg = _align(3 * wb, 256)
        ef.off_su = ef.off_sg + _align(sgu, 256)
        ef.off_sd = ef.off_su + _align(sgu, 256)
        ef.off_tail = ef.off_sd + _align(sd, 256)
        end = ef.off_tail
    elif fmt == "nvfp4":
        wb = H * F // 2
        ef.off_gate, ef.off_up, ef.off_down = 0, wb, 2 * wb
        sgu = quant.sf_atom_size(F, H)
        sd = quant.sf_atom_size(H, F)
        ef.off_sg = _align(3 * wb, 512)
        ef.off_su = ef.off_sg + sgu
        ef.off_sd = ef.off_su + sgu
        ef.off_tail = ef.off_sd + sd
        end = ef.off_tail + 32
    elif fmt == "gguf_q4_k":
        if H % 256 or F % 256:
            raise ValueError("Q4_K experts need hidden and intermediate sizes that are multiples of 256")
        wb = H * F // 256 * 144
        ef.off_gate, ef.off_up, ef.off_down = 0, wb, 2 * wb
        ef.off_sg = ef.off_su = ef.off_sd = ef.off_tail = 3 * wb
        end = 3 * wb
    else:
        raise ValueError(fmt)
    ef.stride = _align(end, 4096)
    return ef


F32_SPLIT_MIN_ROWS = 128  # rows from which an fp32 matrix (the router) runs as a split-bf16 tensor-core GEMM instead of the CUDA-core SGEMM
TC_MOE_MIN_ROWS = 16      # rows per step from which the routed experts run on the tensor-core grouped GEMM
# router projection + top-k in one launch for decode-sized steps (switch: LSB_ROUTER_FUSED=1).  Off by default: measured on the
# GLM-5.3-Flash shape the fused kernel (one block per expert, last block selects) gives 7.21 ms per decode step against 7.12 ms for
# the split-K GEMV + top-k pair, whose second launch already overlaps the first through programmatic dependent launch
ROUTER_FUSED = os.environ.get("LSB_ROUTER_FUSED", "0") != "0"
# LSB_KDA_CHUNKED=0: prefill chunks of one sequence (>= 128 rows) run the KDA recurrence token by token instead of chunk-parallel
# (kda_chunk_prep / kda_chunk_scan).  Chunk-parallel is the default: on a B200 its logits are as close to the fp32 oracle as the token
# recurrence's (1.1e-3 .. 1.8e-3 relative on the tiny model against 1.1e-3 .. 8.6e-3) and a 2048-token chunk is faster.
KDA_CHUNKED = os.environ.get("LSB_KDA_CHUNKED", "1") not in ("", "0")
# LSB_MOE_BLOCK_SCALED=1: many-row steps over NVFP4 experts quantise the activations to NVFP4 (one scale per 16 elements and
# one per row) and run the block-scaled tensor-core kernel (4-bit x 4-bit) instead of expanding the weights to fp16
# LSB_INDEXER_TC=0: score prefill chunks with the CUDA-core indexer kernel instead of the tcgen05 one
INDEXER_TC = os.environ.get("LSB_INDEXER_TC", "1") not in ("", "0")
# steps of few rows over long index rows (more than TOPK_SPLIT_MIN_ENTRIES entries of capacity): the top-k of a row is spread
# over many blocks (five small launches) instead of one block per row
# few-row steps over long index rows (capacity of at least INDEXER_F8_MIN_ENTRIES entries): FP8 x FP8 scoring on the tensor cores
# straight over the cached keys, the query heads quantised to E4M3 per head (scores move by about a percent)
INDEXER_F8 = os.environ.get("LSB_INDEXER_F8", "1") not in ("", "0")
INDEXER_F8_MIN_ENTRIES = int(os.environ.get("LSB_INDEXER_F8_MIN_ENTRIES", "32768"))
TOPK_SPLIT = os.environ.get("LSB_TOPK_SPLIT", "1") not in ("", "0")
TOPK_SPLIT_MIN_ENTRIES = 16384
TOPK_SPLIT_MAX_ROWS = 64
MOE_BLOCK_SCALED = os.environ.get("LSB_MOE_BLOCK_SCALED", "0") not in ("", "0")
# LSB_MHC_CLUSTER=0: decode-sized hyper-connection passes fall back to the two-launch path (partials + last-block finalize, contraction)
MHC_CLUSTER = os.environ.get("LSB_MHC_CLUSTER", "1") not in ("", "0")
# rows of a step up to which the cluster kernel (one cluster per row) is used; above it the partial + last-block-finalize kernels, which
# tile better over many rows (32 rows on a B200: 32.6 us per pass against 55.2 us for 32 clusters)
MHC_CLUSTER_MAX_ROWS = int(os.environ.get("LSB_MHC_CLUSTER_MAX_ROWS", "8"))
# ablation switches of the two folds of the cluster kernel (router behind, MoE combine in front)
MHC_FOLD_ROUTER = os.environ.get("LSB_MHC_FOLD_ROUTER", "0") not in ("", "0")
MHC_FOLD_COMBINE = os.environ.get("LSB_MHC_FOLD_COMBINE", "0") not in ("", "0")
# LSB_MOE_RUN_GU / LSB_MOE_RUN_DN: rows of n % 32 per block of the pair-mode NVFP4 expert kernels (gate/up: 8, 4, 2; down: 16, 8, 4); 0 = by GPU count
MOE_RUN_GU = int(os.environ.get("LSB_MOE_RUN_GU", "0") or 0)
MOE_RUN_DN = int(os.environ.get("LSB_MOE_RUN_DN", "0") or 0)
# LSB_COMM_XCHG: how few-row steps do the fused all-reduce - 0 the producer's last block pushes the partial, 1 the consuming kernel
# exchanges it with one flag per CTA, 2 (default) the consuming kernel exchanges flag-in-data words (no fence, no flag, no barrier)
COMM_XCHG = int(os.environ.get("LSB_COMM_XCHG", "2") or 0)


def _dequant_ggml(t: int, dev_rows: torch.Tensor, N: int, K: int) -> torch.Tensor:
    """fp32 [N, K] of a matrix stored in the device layout of GGUF block type ``t`` (CPU codec: the oracle of the GPU decoders)."""
    from ..formats import gguf as _gguf
    raw = _gguf.from_device_layout(t, dev_rows.detach().cpu().numpy(), N, K)
    return torch.from_numpy(_gguf.dequantize(t, raw, N * K)).view(N, K).to(dev_rows.device)


def _dequant_q4k(raw: torch.Tensor, N: int, K: int) -> torch.Tensor:
    from ..formats import gguf as _gguf
    out = _gguf.dequantize(_gguf.GGML_TYPES["Q4_K"], raw.detach().cpu().numpy().reshape(-1), N * K)
    return torch.from_numpy(out).view(N, K).to(raw.device)


class TcScratch:
    """Per-device scratch of the tensor-core GEMM: split-K partials and the kernel's error word."""
    _inst: Dict[int, "TcScratch"] = {}

    def __init__(self, device):
        self.cap = 16 << 20
        self.partial = torch.empty(self.cap, dtype=torch.float32, device=device)
        self.err = torch.zeros(1, dtype=torch.int32, device=device)

    @classmethod
    def get(cls, device) -> "TcScratch":
        idx = torch.device(device).index or 0
        if idx not in cls._inst:
            cls._inst[idx] = cls(device)
        return cls._inst[idx]


def fp8_scale_atoms(scales: torch.Tensor) -> Optional[torch.Tensor]:
    """UE8M0 scale atoms of an FP8 matrix for the block-scaled tensor-core kernel from its fp32 128 x 128 block scales
    (``[..., rows / 128, K / 128]``): every block becomes one 512-byte atom filled with the scale's exponent byte.  None when a
    scale is not a positive power of two (the instruction's scales have no mantissa; DeepSeek-V3.1+ checkpoints store powers of
    two, others stay on the fp16-operand path)."""
    bits = scales.contiguous().view(torch.int32)
    if bool(((bits & 0x7FFFFF) != 0).any()) or bool((bits <= 0).any()):
        return None
    e = ((bits >> 23) & 0xFF).to(torch.uint8)
    return e.reshape(*e.shape[:-2], -1, 1).expand(*e.shape[:-2], e.shape[-2] * e.shape[-1], 512).contiguous()


class QLinear:
    """A weight matrix [N, K] in a device storage format, applied to bf16 activations.
    Up to 4 rows (decode) stream the weights through the CUDA-core GEMV; larger row counts with
    bf16 weights run on the tcgen05 tensor-core GEMM."""

    def __init__(self, fmt: str, N: int, K: int, w: torch.Tensor, scales: Optional[torch.Tensor] = None, alpha: float = 1.0):
        self.fmt, self.N, self.K, self.w, self.scales, self.alpha = fmt, N, K, w, scales, alpha

    @staticmethod
    def from_float(wf: torch.Tensor, fmt: str, device) -> "QLinear":
        N, K = wf.shape
        wf = wf.to(device)
        if fmt == "bf16":
            return QLinear("bf16", N, K, wf.to(torch.bfloat16).contiguous())
        if fmt == "f32":
            return QLinear("f32", N, K, wf.float().contiguous())
        if fmt == "fp8_e4m3":
            q, s = quant.quantize_fp8_block(wf)
            return QLinear("fp8_e4m3", N, K, q, s)
        if fmt == "nvfp4":
            q, a, gs = quant.quantize_nvfp4(wf)
            return QLinear("nvfp4", N, K, q, a, gs)
        if fmt == "gguf_q4_k":
            from ..formats import gguf as _gguf
            raw = _gguf.quantize(_gguf.GGML_TYPES["Q4_K"], wf.float().cpu().numpy())
            return QLinear("gguf_q4_k", N, K, torch.from_numpy(raw).to(device).view(N, K // 256 * 144))
        if fmt in ("gguf_q6_k", "gguf_q8_0"):
            from ..formats import gguf as _gguf
            t = GGML_OF[fmt]
            return QLinear.from_ggml(t, _gguf.quantize(t, wf.float().cpu().numpy()), N, K, device)
        raise ValueError(fmt)

    @staticmethod
    def from_ggml(t: int, raw, N: int, K: int, device) -> "QLinear":
        """File-order GGUF blocks of type ``t`` (Q4_K, Q5_K, Q6_K, Q8_0) -> the device layout of that type, values untouched."""
        from ..formats import gguf as _gguf
        import numpy as _np
        raw = raw.cpu().numpy() if isinstance(raw, torch.Tensor) else _np.asarray(raw)
        d = _gguf.to_device_layout(t, raw, N, K)
        return QLinear(_gguf.DEVICE_NATIVE[t], N, K, torch.from_numpy(_np.ascontiguousarray(d)).to(device))

    @staticmethod
    def random(N: int, K: int, fmt: str, device, std: float = 0.02, gen=None) -> "QLinear":
        """Random-init directly in storage format (no fp32 master copy)."""
        if fmt == "bf16":
            w = torch.empty(N, K, dtype=torch.bfloat16, device=device)
            w.normal_(0.0, std, generator=gen)
            return QLinear("bf16", N, K, w)
        if fmt == "f32":
            w = torch.empty(N, K, dtype=torch.float32, device=device)
            w.normal_(0.0, std, generator=gen)
            return QLinear("f32", N, K, w)
        if fmt == "fp8_e4m3":
            w = torch.empty(N, K, dtype=torch.uint8, device=device)
            w.random_(0, 256, generator=gen)
            w &= 0xBF   # keep |value| <= 1.875: clear the top exponent bit, never a NaN code
            # block scales are powers of two (the UE8M0 convention of DeepSeek-V3.1+ checkpoints): the nearest one to std / 0.6
            s = torch.full(((N + 127) // 128, (K + 127) // 128), 2.0 ** round(math.log2(std / 0.6)), dtype=torch.float32, device=device)
            return QLinear("fp8_e4m3", N, K, w, s)
        if fmt == "nvfp4":
            w = torch.empty(N, K // 2, dtype=torch.uint8, device=device)
            a = torch.empty(quant.sf_atom_size(N, K), dtype=torch.uint8, device=device)
            gs = quant.random_nvfp4_(w, a, gen) * (std / 0.02)
            return QLinear("nvfp4", N, K, w, a, gs)
        if fmt == "gguf_q4_k":
            # random quants and 6-bit scales; d / dmin fixed so that weights ~ U(-c, c) with standard deviation `std`
            blocks = torch.empty(N * K // 256, 144, dtype=torch.uint8, device=device)
            blocks.random_(0, 256, generator=gen)
            c = std * 3 ** 0.5
            d = torch.tensor([c / 7.5 / 32.0, c / 32.0], dtype=torch.float16).view(torch.uint8).to(device)      # d*sc*q - dmin*m with sc~32, m~32
            blocks[:, :4] = d
            blocks[:, 4:16] = (blocks[:, 4:16] & 0x1F) | 0x10      # scales and mins in 16..31, top bits clear
            return QLinear("gguf_q4_k", N, K, blocks.view(N, K // 256 * 144))
        if fmt in ("gguf_q5_k", "gguf_q6_k", "gguf_q8_0"):
            # random quants in file order with fixed block scales, then the device layout
            c = std * 3 ** 0.5
            if fmt == "gguf_q5_k":
                blocks = torch.empty(N * K // 256, 176, dtype=torch.uint8, device=device)
                blocks.random_(0, 256, generator=gen)
                blocks[:, :4] = torch.tensor([c / 15.5 / 32.0, c / 32.0], dtype=torch.float16).view(torch.uint8).to(device)
                blocks[:, 4:16] = (blocks[:, 4:16] & 0x1F) | 0x10
            elif fmt == "gguf_q6_k":
                blocks = torch.empty(N * K // 256, 210, dtype=torch.uint8, device=device)
                blocks.random_(0, 256, generator=gen)
                blocks[:, 192:208] = (blocks[:, 192:208] & 0x3F) | 0x20          # int8 scales 32..95
                blocks[:, 208:210] = torch.tensor([c / 32.0 / 64.0], dtype=torch.float16).view(torch.uint8).to(device)
            else:
                blocks = torch.empty(N * K // 32, 34, dtype=torch.uint8, device=device)
                blocks.random_(0, 256, generator=gen)
                blocks[:, :2] = torch.tensor([c / 127.0], dtype=torch.float16).view(torch.uint8).to(device)
            return QLinear.from_ggml(GGML_OF[fmt], blocks, N, K, device)
        raise ValueError(fmt)

    _tiles: Dict[tuple, dict] = {}
    _x16: Dict[int, torch.Tensor] = {}

    @classmethod
    def _dense_tiles(cls, device, M: int) -> dict:
        """Tile description of a dense [M, K] operand for the grouped tensor-core kernel (constant per M) and the shared
        fp16 staging buffer for the activations."""
        idx = torch.device(device).index or 0
        key = (idx, M)
        if key not in cls._tiles:
            bn = 32 if M <= 32 else (64 if M <= 64 else 128)
            n = (M + bn - 1) // bn
            i32 = dict(dtype=torch.int32, device=device)
            r0 = torch.arange(n, **i32) * bn
            cls._tiles[key] = {"bn": bn, "n": n, "te": torch.zeros(n, **i32), "tr": r0, "tn": torch.clamp(M - r0, max=bn).int(),
                               "cnt": torch.tensor([n, M], **i32), "ident": torch.arange(M, **i32), "slot0": torch.zeros(1, **i32)}
        t = cls._tiles[key]
        need = M * 32768
        if idx not in cls._x16 or cls._x16[idx].numel() < need:
            cls._x16[idx] = torch.empty(max(need, 4096 * 32768), dtype=torch.float16, device=device)
        t["x16"] = cls._x16[idx]
        return t

    _f32s: Dict[int, torch.Tensor] = {}

    @classmethod
    def _f32_scratch(cls, device, n: int) -> torch.Tensor:
        idx = torch.device(device).index or 0
        if idx not in cls._f32s or cls._f32s[idx].numel() < n:
            cls._f32s[idx] = torch.empty(n, dtype=torch.float32, device=device)
        return cls._f32s[idx][:n]

    _bf16: Dict[int, torch.Tensor] = {}

    @classmethod
    def _bf16_scratch(cls, device, n: int) -> torch.Tensor:
        idx = torch.device(device).index or 0
        if idx not in cls._bf16 or cls._bf16[idx].numel() < n:
            cls._bf16[idx] = torch.empty(n, dtype=torch.bfloat16, device=device)
        return cls._bf16[idx]

    _bsbuf: Dict[tuple, tuple] = {}

    @classmethod
    def _bs_operand(cls, device, rows: int, ntiles: int, K: int, fp8: bool = False):
        """Scratch for the NVFP4 (or FP8) image of a dense activation operand: packed values, scale atoms, per-row scales."""
        key = (torch.device(device).index or 0, rows, ntiles, K, fp8)
        if key not in cls._bsbuf:
            if len(cls._bsbuf) > 64:
                cls._bsbuf.clear()
            cls._bsbuf[key] = (torch.zeros(rows, K if fp8 else K // 2, dtype=torch.uint8, device=device),
                               torch.zeros(ntiles * (K // (128 if fp8 else 64)) * 512, dtype=torch.uint8, device=device), torch.zeros(rows, device=device))
        return cls._bsbuf[key]

    def bs_scale_atoms(self):
        """FP8 weights: the UE8M0 scale atoms of this matrix (built once), or None when its block scales are not powers of two."""
        if not hasattr(self, "_bs_wsf"):
            self._bs_wsf = fp8_scale_atoms(self.scales.view(torch.float32).reshape((self.N + 127) // 128, (self.K + 127) // 128)) \
                if (self.fmt == "fp8_e4m3" and self.N % 128 == 0 and self.K % 128 == 0) else None
        return self._bs_wsf

    def dequant(self) -> torch.Tensor:
        if self.fmt in ("bf16", "f32"):
            return self.w.float()
        if self.fmt == "fp8_e4m3":
            return quant.dequantize_fp8_block(self.w, self.scales)
        if self.fmt in GGML_OF:
            return _dequant_ggml(GGML_OF[self.fmt], self.w, self.N, self.K)
        return quant.dequantize_nvfp4(self.w, self.scales, self.alpha, self.N, self.K)

    def nbytes(self) -> int:
        return self.w.numel() * self.w.element_size() + (self.scales.numel() * self.scales.element_size() if self.scales is not None else 0)

    def __call__(self, out: torch.Tensor, x: torch.Tensor, M: int, ldx: Optional[int] = None, ldo: Optional[int] = None,
                 bias: Optional[torch.Tensor] = None, comm: Optional[int] = None):
        """out[M, N] = x[M, K] @ W^T.  ``comm`` (address of a PeerComm struct) turns the store into the
        push half of a fused cross-rank all-reduce (row-parallel layers)."""
        ldx = ldx if ldx is not None else self.K
        ldo = ldo if ldo is not None else self.N
        ob = 1 if out.dtype == torch.bfloat16 else 0
        if comm is not None and M not in (1, 2, 4) and not (self.fmt == "bf16" and M >= 8 and bias is None and not ob):
            # no fused epilogue for this shape / format: compute the partial locally, then push it to the peers with a copy kernel
            if ob:
                raise RuntimeError("the cross-rank reduction needs an fp32 partial")
            self(out, x, M, ldx, ldo, bias, None)
            nat.call("lsb_comm_push_rows", out, M, self.N, ldo, comm)
            return
        if self.fmt == "bf16" and M >= 8:
            sc = TcScratch.get(self.w.device)
            nat.call("lsb_gemm_bf16_tc", out, x, self.w, bias, M, self.N, self.K, ldx, self.K, ldo, ob, sc.partial, sc.cap, sc.err, comm)
        elif (self.fmt == "nvfp4" and MOE_BLOCK_SCALED and M >= 16 and comm is None and bias is None and ldx == self.K and self.K % 256 == 0
              and self.K <= 8192 and self.N % 128 == 0):
            # many rows over NVFP4 weights, block-scaled mode: the rows are quantised to NVFP4 and both operands stay 4-bit
            t = QLinear._dense_tiles(self.w.device, M)
            q, sf, al = QLinear._bs_operand(self.w.device, t["n"] * t["bn"], t["n"], self.K)
            nat.call("lsb_quant_nvfp4_tiles", x, 2, None, t["tr"], t["tn"], t["cnt"], 1, self.K, t["bn"], t["n"], q, sf, al)
            nat.call("lsb_gemm_nvfp4_bs", out, q, sf, al, self.w, self.scales, self.alpha, self.N, self.K, ldo, ob, t["tr"], t["tn"], t["cnt"],
                     t["bn"], t["n"], TcScratch.get(self.w.device).err)
        elif (self.fmt == "fp8_e4m3" and MOE_BLOCK_SCALED and M >= 16 and comm is None and bias is None and ldx == self.K and self.K % 128 == 0
              and self.K <= 8192 and self.N % 128 == 0 and self.bs_scale_atoms() is not None):
            # many rows over FP8 weights, block-scaled mode: the rows are quantised to FP8 with power-of-two group scales, both
            # operands go to the tensor core as they are (kind::mxf8f6f4.block_scale)
            t = QLinear._dense_tiles(self.w.device, M)
            q, sf, al = QLinear._bs_operand(self.w.device, t["n"] * t["bn"], t["n"], self.K, fp8=True)
            nat.call("lsb_quant_fp8_tiles", x, 2, None, t["tr"], t["tn"], t["cnt"], 1, self.K, t["bn"], t["n"], q, sf, al)
            nat.call("lsb_gemm_fp8_bs", out, q, sf, al, self.w, self._bs_wsf, self.N, self.K, ldo, ob, t["tr"], t["tn"], t["cnt"],
                     t["bn"], t["n"], TcScratch.get(self.w.device).err)
        elif (self.fmt in ("fp8_e4m3", "nvfp4", "gguf_q4_k") and M >= 16 and comm is None and bias is None and ldx == self.K and self.K % 64 == 0
              and self.N % 128 == 0 and (self.fmt != "fp8_e4m3" or self.K % 128 == 0) and (self.fmt != "gguf_q4_k" or self.K % 256 == 0)):
            # many rows over quantised weights: de-quantisation fused into the tcgen05 operand pipeline
            t = QLinear._dense_tiles(self.w.device, M)
            nat.call("lsb_moe_tc_gather", x, t["ident"], t["cnt"], t["x16"], M, 1, self.K)
            nat.call("lsb_gemm_q_tc", out, t["x16"], self.w, self.scales, EXPERT_FMT[self.fmt], M, self.N, self.K, ldo, ob,
                     self.alpha if self.fmt == "nvfp4" else 1.0, t["te"], t["tr"], t["tn"], t["cnt"], t["ident"], t["slot0"], t["bn"], t["n"],
                     TcScratch.get(self.w.device).err)
        elif self.fmt == "bf16":
            nat.call("lsb_gemv_bf16", out, x, self.w, bias, M, self.N, self.K, ldx, self.K, ldo, 1.0, ob, comm)
        elif self.fmt == "f32" and M >= F32_SPLIT_MIN_ROWS and bias is None and not ob and ldx == self.K and ldo == self.N and self.K % 64 == 0:
            # many rows over an fp32 matrix (the router of a prefill chunk): w = hi + lo with both halves bf16 (exact to 2^-17
            # relative), ONE tensor-core GEMM over the stacked [hi; lo] rows, then the two halves of the result are added
            if getattr(self, "_hilo", None) is None:
                hi = self.w.to(torch.bfloat16)
                lo = (self.w - hi.float()).to(torch.bfloat16)
                self._hilo = torch.cat([hi, lo], 0).contiguous()
            tmp = QLinear._f32_scratch(self.w.device, M * 2 * self.N).view(M, 2 * self.N)
            sc = TcScratch.get(self.w.device)
            nat.call("lsb_gemm_bf16_tc", tmp, x, self._hilo, None, M, 2 * self.N, self.K, ldx, self.K, 2 * self.N, 0, sc.partial, sc.cap, sc.err, None)
            torch.add(tmp[:, : self.N], tmp[:, self.N:], out=out[:M].view(M, self.N) if out.dim() == 2 else out.view(-1)[: M * self.N].view(M, self.N))
        elif self.fmt == "f32":
            nat.call("lsb_gemv_f32w", out, x, self.w, bias, M, self.N, self.K, ldx, self.K, ldo, 1.0, ob)
        elif self.fmt == "gguf_q4_k":
            nat.call("lsb_gemv_q4k", out, x, self.w, bias, M, self.N, self.K, ldx, ldo, 1.0, ob, comm)
        elif self.fmt in GGML_OF:
            if M >= 16 and comm is None and ldx == self.K:
                # many rows: expand the blocks to bf16 once per call (scratch shared by all layers) and run the tensor-core GEMM
                scr = QLinear._bf16_scratch(self.w.device, self.N * self.K)
                nat.call("lsb_gguf_dequant_bf16", scr, self.w, GGML_OF[self.fmt], self.N, self.K)
                sc = TcScratch.get(self.w.device)
                nat.call("lsb_gemm_bf16_tc", out, x, scr, bias, M, self.N, self.K, ldx, self.K, ldo, ob, sc.partial, sc.cap, sc.err, None)
            else:
                nat.call("lsb_gemv_gguf", out, x, self.w, GGML_OF[self.fmt], bias, M, self.N, self.K, ldx, ldo, 1.0, ob, comm)
        elif self.fmt == "fp8_e4m3":
            nat.call("lsb_gemv_fp8b", out, x, self.w, self.scales, bias, M, self.N, self.K, ldx, ldo, 1.0, ob, comm)
        else:
            nat.call("lsb_gemv_nvfp4", out, x, self.w, self.scales, bias, M, self.N, self.K, ldx, ldo, self.alpha, ob, comm)


@dataclass
class MlaOffsets:
    qa: int = 0
    kv: int = 0
    idx_k: int = -1
    idx_w: int = -1
    idx_gate: int = -1
    total: int = 0
    q_idx: int = -1      # offset of indexer q inside the fused q_b output
    qb_total: int = 0


class ExpertArena:
    """Slotted expert storage of one MoE layer.  ``slot_of`` maps expert id (routed 0..E-1, shared
    E..E+n_shared-1) to a slot or -1."""

    def __init__(self, ef: ExpertFmt, n_slots: int, n_experts_total: int, device):
        self.ef = ef
        self.n_slots = n_slots
        self.data = torch.empty(n_slots, ef.stride, dtype=torch.uint8, device=device)
        self.slot_of = torch.full((n_experts_total,), -1, dtype=torch.int32, device=device)

    def slot_view(self, slot: int) -> torch.Tensor:
        return self.data[slot]

    def write_expert(self, slot: int, gate: QLinear, up: QLinear, down: QLinear):
        ef, v = self.ef, self.data[slot]

        def put(off, t):
            b = t.contiguous().view(torch.uint8).reshape(-1)
            v[off: off + b.numel()] = b

        put(ef.off_gate, gate.w); put(ef.off_up, up.w); put(ef.off_down, down.w)
        if gate.scales is not None:
            put(ef.off_sg, gate.scales); put(ef.off_su, up.scales); put(ef.off_sd, down.scales)
        if ef.fmt == 2:
            put(ef.off_tail, torch.tensor([gate.alpha, up.alpha, down.alpha], dtype=torch.float32, device=v.device))

    def bs_scale_atoms(self):
        """FP8 arenas: (atoms [n_slots, bytes], byte offsets of the gate / up / down matrices' atoms) for the block-scaled
        tensor-core kernel, derived once from the slots' 128 x 128 block scales; None when the format is another one, the
        widths are not multiples of 128 or a scale is not a power of two.  Built from the slots as they are NOW: arenas whose
        slots change (expert streaming) must not use it."""
        if not hasattr(self, "_bs_wsf"):
            self._bs_wsf = None
            ef = self.ef
            if ef.fmt == 1 and ef.H % 128 == 0 and ef.F % 128 == 0:
                ngu, nd = (ef.F // 128) * (ef.H // 128), (ef.H // 128) * (ef.F // 128)
                parts = []
                for off, n, shape in ((ef.off_sg, ngu, (ef.F // 128, ef.H // 128)), (ef.off_su, ngu, (ef.F // 128, ef.H // 128)),
                                      (ef.off_sd, nd, (ef.H // 128, ef.F // 128))):
                    sc = self.data[:, off: off + 4 * n].contiguous().view(torch.float32).view(self.n_slots, *shape)
                    a = fp8_scale_atoms(sc)
                    if a is None:
                        parts = None
                        break
                    parts.append(a.reshape(self.n_slots, -1))
                if parts is not None:
                    self._bs_wsf = (torch.cat(parts, 1).contiguous(), 0, ngu * 512, 2 * ngu * 512)
        return self._bs_wsf

    def read_expert(self, slot: int, fmt: str):
        """Dequantised (gate, up, down) fp32 matrices of a slot (tests / oracle)."""
        ef, v = self.ef, self.data[slot]
        H, F = ef.H, ef.F
        out = []
        for nm, (N, K), ow, os_ in (("gate", (F, H), ef.off_gate, ef.off_sg), ("up", (F, H), ef.off_up, ef.off_su),
                                   ("down", (H, F), ef.off_down, ef.off_sd)):
            if fmt == "bf16":
                out.append(v[ow: ow + N * K * 2].view(torch.bfloat16).view(N, K).float())
            elif fmt in GGML_OF:
                from ..formats import gguf as _gguf
                t = GGML_OF[fmt] if (nm != "down" or not ef.fmt_down1) else GGML_OF[_FMT_NAME[ef.fmt_down1 - 1]]
                rb = _gguf.device_row_bytes(t, K)
                out.append(_dequant_ggml(t, v[ow: ow + N * rb].view(N, rb), N, K))
            elif fmt == "fp8_e4m3":
                nb = ((N + 127) // 128) * ((K + 127) // 128)
                s = v[os_: os_ + nb * 4].view(torch.float32).view((N + 127) // 128, (K + 127) // 128)
                out.append(quant.dequantize_fp8_block(v[ow: ow + N * K].view(N, K), s))
            else:
                tail = v[ef.off_tail: ef.off_tail + 12].view(torch.float32)
                i = {"gate": 0, "up": 1, "down": 2}[nm]
                out.append(quant.dequantize_nvfp4(v[ow: ow + N * K // 2].view(N, K // 2), v[os_: os_ + quant.sf_atom_size(N, K)],
                                                  float(tail[i]), N, K))
        return out


class Workspace:
    """Static activation buffers for steps of up to ``R`` rows."""

    def __init__(self, m: "DeviceModel", R: int, n_logit_rows: int, max_ctx: int):
        cfg, dev = m.cfg, m.device
        f32, b16, i32 = torch.float32, torch.bfloat16, torch.int32
        H, n = cfg.hidden, cfg.hc_mult
        self.R = R

        def z(*shape, dtype=f32):
            return torch.zeros(*shape, dtype=dtype, device=dev)

        # step inputs: one packed int32 buffer so a step needs a single host->device copy
        self.inp = z(9, R, dtype=i32)
        self.inp[1].fill_(-1)
        (self.tok, self.row_seq, self.row_pos, self.row_len, self.row_slot, self.n_entries,
         self.seq_row0, self.seq_nrows, self.seq_slot) = (self.inp[j] for j in range(9))
        # activations
        self.x = z(R, H, dtype=b16)
        self.mtp_cat = z(R, 2 * H, dtype=b16) if m.mtp_layers else None       # [RMSNorm(embedding) ; RMSNorm(stream)] of an MTP block
        self.sub = z(R, H)
        self.resid = z(R, n, H)
        self.post = z(R, n); self.comb = z(R, n, n)
        self.part = z(R, max(1, H // 32), 36)
        self.hc_done = z(max(R, 1), dtype=i32)
        self.hc_pre = z(max(R, 1), 8)
        self.proj = z(R, m.max_proj)
        C = m.Hk * cfg.kda_head_dim
        self.kda_out = z(R, max(C, 1), dtype=b16)
        # many-row KDA path: q / k / v->o / decay / gate [R, C] and beta [R, heads], fp32
        # KDA chunk path: 5 + 2 per-channel arrays, beta, the bf16 (hi | lo) gate activations and an error word
        self.router_done = torch.zeros(1, dtype=i32, device=dev)
        self.row_store = torch.zeros(R, dtype=i32, device=dev)          # context-parallel KV: shard index of each new row (-1: not ours)
        self.row_len_local = torch.zeros(R, dtype=i32, device=dev)      # ... and the number of visible positions this rank stores
        self.kda_scratch = z(7 * R * C + R * m.Hk + 2 * R * m.cfg.kda_rank + 16) if (C > 0 and R >= 8) else None
        # workspace of the chunk-parallel KDA recurrence (W, tril(B) and the chunk decays of every 64-token chunk); opt-in
        self.kda_chunk_ws = z(((R + 63) // 64) * m.Hk * (2 * 64 * 64 + 128)) if (KDA_CHUNKED and C > 0 and R >= 128) else None
        Hh = m.Hh
        self.q_c = z(R, max(cfg.q_lora, 1), dtype=b16)
        self.qproj = z(R, m.max_qb, dtype=b16)
        self.q_abs = z(R, Hh, cfg.kv_lora + cfg.qk_rope, dtype=b16)
        self.o_lat = z(R, Hh, cfg.kv_lora, dtype=b16)
        # KV splits: enough blocks for two per SM.  Blocks per query row follow the kernel variant lsb_mla_decode picks (one block
        # serves four 16-head groups above 32 heads, two above 16)
        hb = (Hh + 63) // 64 if Hh > 32 else ((Hh + 31) // 32 if Hh > 16 else 1)
        self.NS = max(1, min(32, 296 // max(1, R * hb)))
        self.o_part = z(R, Hh, self.NS, cfg.kv_lora)
        self.ml_part = z(R, Hh, self.NS, 2)
        self.attn_v = z(R, Hh * cfg.v_head, dtype=b16)
        if cfg.has_indexer:
            P = cfg.index_kpool
            self.max_entries = (max_ctx + P - 1) // P
            self.scores = z(R, self.max_entries)
            self.sel_ld = cfg.index_topk + P
            self.sel_idx = z(R, self.sel_ld, dtype=i32)
            self.sel_cnt = z(R, dtype=i32)
            self.q_idx = z(R, cfg.index_n_heads, cfg.index_head_dim, dtype=b16)
            self.topk_scratch = None
            if TOPK_SPLIT and R <= TOPK_SPLIT_MAX_ROWS and self.max_entries > TOPK_SPLIT_MIN_ENTRIES:
                nbytes = int(nat.call("lsb_indexer_topk_split_scratch", R, self.max_entries))
                self.topk_scratch = z((nbytes + 3) // 4, dtype=i32)         # zeroed once; every launch leaves it zeroed
            # tensor-core scoring of single-sequence chunks: the sequence's index keys as a dense bf16 operand + their scales
            # (single-row decode steps do not use that path: at 262k entries key gather + GEMM take 184 us against 88 us on the CUDA cores)
            pe = m.page // P
            self.idx_f8 = (INDEXER_F8 and R < 64 and self.max_entries >= INDEXER_F8_MIN_ENTRIES and cfg.index_head_dim == 128
                           and cfg.index_n_heads <= 64 and 8 <= pe <= 128 and pe & (pe - 1) == 0)
            self.idx_tc = (INDEXER_TC and R >= 64 and cfg.index_head_dim == 128 and 256 % cfg.index_n_heads == 0)
            if self.idx_tc:
                self.idx_kbf_rows = (self.max_entries + 127) // 128 * 128
                self.idx_kbf = z(self.idx_kbf_rows, 128, dtype=b16)
                self.idx_kscale = z(self.idx_kbf_rows)
            self.ne_hint, self.single_seq = 0, False
            self.idx_w = z(R, cfg.index_n_heads)
            self.kstash = z(R, cfg.index_head_dim, dtype=b16)
        # FFN
        F = max(m.Fd, 1)
        self.gu = z(R, 2 * F)
        self.act_d = z(R, F, dtype=b16)
        if cfg.n_routed > 0:
            S = cfg.top_k + cfg.n_shared
            E_total = cfg.n_routed + cfg.n_shared
            self.S = S
            self.logits_r = z(R, cfg.n_routed)
            self.ids = z(R, S, dtype=i32); self.wts = z(R, S)
            self.max_groups = min(R * S, (R * S + 3) // 4 + E_total)
            self.group_expert = z(self.max_groups, dtype=i32); self.group_n = z(self.max_groups, dtype=i32)
            self.group_pairs = z(self.max_groups * 4, dtype=i32); self.n_groups = z(1, dtype=i32)
            self.counts = z(2 * E_total + 2, dtype=i32)
            self.act = z(R * S, cfg.moe_inter, dtype=b16)
            self.y = z(R * S, H)
            self.miss = z(1, dtype=i32)
            # tensor-core grouped path (many rows): expert-sorted fp16 operands and the device-built tile list
            self.tc_ok = R >= TC_MOE_MIN_ROWS and H % 64 == 0 and H % 128 == 0 and m.Fe % 128 == 0
            if self.tc_ok:
                P = R * S
                avg = P / max(1, min(E_total, P))
                self.tc_bn = 32 if avg <= 32 else (64 if avg <= 96 else 128)
                self.tc_tiles = P // self.tc_bn + E_total + 1
                self.tc_sorted = z(P, dtype=i32)
                self.tc_tile_e = z(self.tc_tiles, dtype=i32); self.tc_tile_r0 = z(self.tc_tiles, dtype=i32)
                self.tc_tile_n = z(self.tc_tiles, dtype=i32); self.tc_cnt = z(2, dtype=i32)
                # block-scaled path (NVFP4 experts): both operands stay 4-bit, the activations are quantised in tile order
                fmts = {L["arena"].ef.fmt for L in m.layers if L.get("arena") is not None}
                self.bs_can = fmts == {2} and H % 256 == 0 and m.Fe % 256 == 0 and H <= 8192 and m.Fe <= 8192
                # ... or FP8 experts whose block scales are powers of two (FP8 activations with UE8M0 group scales); not with a capped
                # expert cache, whose slots change under the scale atoms
                self.bs_fp8 = (fmts == {1} and H % 128 == 0 and m.Fe % 128 == 0 and H <= 8192 and m.Fe <= 8192 and m.streamer is None
                               and all(L["arena"].bs_scale_atoms() is not None for L in m.layers if L.get("arena") is not None))
                self.bs_can = self.bs_can or self.bs_fp8
                self.bs_ok = False
                self._m, self._z = m, z
        # outputs
        self.n_logit_rows = n_logit_rows
        self.logits = z(n_logit_rows, m.V_local)
        self.amax_part = torch.zeros(n_logit_rows, 64, dtype=torch.int64, device=dev)
        self.out_tok = z(n_logit_rows, dtype=i32)
        self.out_val = z(n_logit_rows)

        if getattr(self, "tc_ok", False):
            self.set_block_scaled(MOE_BLOCK_SCALED)

    def set_block_scaled(self, on: bool) -> bool:
        """Switch this workspace's many-row expert path between fp16 activations (weights expanded in the operand pipeline) and NVFP4
        activations on the block-scaled tensor-core kernel.  The buffers of a path are allocated the first time it is switched on;
        not while a CUDA graph that uses the workspace exists.  Returns whether the block-scaled path is now active."""
        if not getattr(self, "tc_ok", False):
            return False
        on = bool(on) and self.bs_can
        m, z, H = self._m, self._z, self._m.cfg.hidden
        if on and not hasattr(self, "bs_xq"):
            rows = self.tc_tiles * self.tc_bn
            u8 = torch.uint8
            vb, ak = (1, 128) if self.bs_fp8 else (2, 64)          # values per byte, reduction elements per scale atom
            self.bs_xq = z(rows, H // vb, dtype=u8); self.bs_xsf = z(self.tc_tiles * (H // ak) * 512, dtype=u8); self.bs_xa = z(rows)
            self.bs_act = z(rows, m.Fe, dtype=torch.float16)
            self.bs_aq = z(rows, m.Fe // vb, dtype=u8); self.bs_asf = z(self.tc_tiles * (m.Fe // ak) * 512, dtype=u8); self.bs_aa = z(rows)
        if not on and not hasattr(self, "tc_xs"):
            P = self.tc_sorted.shape[0]
            self.tc_xs = z(P, H, dtype=torch.float16)
            self.tc_act = z(P, m.cfg.moe_inter, dtype=torch.float16)
        self.bs_ok = on
        return on


class DeviceModel:
    def __init__(self, cfg: ModelConfig, device="cuda", kv_fmt: str = "fp8", page: int = 64, tp_rank: int = 0, tp_size: int = 1,
                 expert_shard: Optional[str] = None):
        """``expert_shard``: how the experts are spread over ``tp_size`` GPUs - ``"ep"`` routed expert e lives whole on GPU e % N (the
        shared expert of layer i on GPU i % N), ``"tp"`` every GPU holds a 1/N slice of EVERY expert (gate / up rows, down columns).
        Both end in the same cross-rank sum.  ``"tp"`` gives every GPU the same work whatever the router picks, which is what a
        decode step wants (with ``"ep"`` a token's 8 experts land 4-0-3-1 on 4 GPUs and the step waits for the fullest one);
        default: ``LSB_EXPERT_SHARD``, else ``"tp"`` whenever the expert width divides into slices of 128."""
        self.cfg, self.device = cfg, torch.device(device)
        if expert_shard is None:
            expert_shard = os.environ.get("LSB_EXPERT_SHARD") or ("tp" if (tp_size > 1 and cfg.n_routed and cfg.moe_inter % (128 * tp_size) == 0) else "ep")
        if expert_shard == "tp" and (tp_size == 1 or cfg.moe_inter % tp_size):
            expert_shard = "ep"
        self.expert_shard = expert_shard
        self.Fe = cfg.moe_inter // tp_size if expert_shard == "tp" else cfg.moe_inter        # expert width held by this GPU
        self.kv_fmt, self.page = kv_fmt, page
        assert page % max(cfg.index_kpool, 1) == 0
        # Tensor / expert parallel layout (one process per GPU): attention heads, KDA heads, dense FFN
        # columns and the LM-head vocabulary are split over the ranks; routed experts are owned by rank
        # e % tp_size, the shared expert of layer i by rank i % tp_size; small projections are replicated.
        self.tp_rank, self.tp_size = tp_rank, tp_size
        for v, nm in ((cfg.n_heads, "n_heads"), (cfg.dense_inter, "dense_inter"), (cfg.vocab, "vocab")):
            assert v % tp_size == 0, f"{nm}={v} not divisible by tp={tp_size}"
        assert cfg.kda_heads % tp_size == 0
        self.Hh = cfg.n_heads // tp_size
        self.Hk = cfg.kda_heads // tp_size
        self.Fd = cfg.dense_inter // tp_size
        self.V_local = cfg.vocab // tp_size
        self._fused = False
        self.dcp = None
        self.idx_identity = False  # the indexer's key cache keeps a page table of its own (row-granular KV tiering: its pages never leave HBM)
        self.skip_layers = frozenset()   # layers whose attention + FFN a step leaves out (self-speculative drafting; never the first or last)
        self.probe = None                # {"prev": bf16 [1, hidden], "sims": fp32 [n_layers]} while layer-input similarities are recorded
        self.aux_capture = None          # {"slots": {layer: column}, "buf": bf16 [rows, n_aux, hidden]}: layer inputs kept for a block draft model
        self.row_tier = None      # RowTiering (runtime/kv_tiering.py) when old KV pages of active sequences live in pinned host memory
        self.streamer = None      # ExpertStreamer when the VRAM expert cache is capped (runtime/streaming.py)
        self.drift = None         # dict: eager steps store every layer's output rows here (input of utils/determinism_probe.py drift)
        self.tq_centroids = None  # TurboQuant reconstruction levels (kv_fmt "tq4")
        self.comm = None          # PeerComm for the fused all-reduces
        self.comm_amax = None     # PeerComm for the argmax exchange
        self.layers: List[dict] = []
        self.mtp_layers: List[dict] = []            # multi-token-prediction blocks (layer ids n_layers ..), see forward_mtp
        self.embed = None
        self.head: Optional[QLinear] = None
        self.final_norm = None
        self.max_proj = 1
        self.max_qb = 1
        self.kv_row_bytes = nat.call("lsb_kv_row_bytes", KV_FMT[kv_fmt], cfg.kv_lora, cfg.qk_rope)
        self.idx_row_bytes = nat.call("lsb_indexer_row_bytes")
        inv = cfg.rope_inv_freq()
        self.inv_freq = torch.tensor(inv if inv else [0.0], dtype=torch.float32, device=self.device)
        inv_i = cfg.rope_inv_freq(cfg.index_rope_dim) if cfg.index_rope_dim else [0.0]
        self.inv_freq_idx = torch.tensor(inv_i, dtype=torch.float32, device=self.device)
        # caches (allocated by alloc_cache)
        self.kv_cache: Dict[int, torch.Tensor] = {}
        self.idx_cache: Dict[int, torch.Tensor] = {}
        self.idx_tail: Dict[int, torch.Tensor] = {}
        self.kda_state: Dict[int, torch.Tensor] = {}
        self.kda_conv: Dict[int, torch.Tensor] = {}
        self.block_table = None
        self.kernel_launches = 0

    def attach_comm(self, comm, comm_amax):
        self.comm, self.comm_amax = comm, comm_amax

    def reduced_expert_view(self, top_k: int) -> "DeviceModel":
        """A second model over the SAME weight tensors that routes to ``top_k`` experts per token (own KV / recurrent caches, to be
        allocated by the engine that takes it): the draft side of self-speculative decoding.  Single-GPU models with fully resident
        experts only - the in-kernel collectives' buffers and the expert streamer's slots belong to the full model's step."""
        import copy
        import dataclasses
        if self.tp_size != 1 or self.streamer is not None:
            raise NotImplementedError("reduced-expert view needs tp_size == 1 and fully resident experts")
        v = copy.copy(self)
        v.cfg = dataclasses.replace(self.cfg, top_k=max(1, min(top_k, self.cfg.top_k)))
        v.kv_cache, v.idx_cache, v.idx_tail, v.kda_state, v.kda_conv = {}, {}, {}, {}, {}
        v.block_table = None
        v.drift = None
        v.kernel_launches = 0
        return v

    def mtp_supported(self) -> bool:
        """Whether this model can run multi-token-prediction blocks on the device: one GPU, a plain residual stream (no
        hyper-connections: their final stream is never materialised un-normalised) and an FP8 / bf16 latent cache."""
        return self.tp_size == 1 and not self.cfg.mhc and self.kv_fmt != "tq4" and self.cfg.n_mtp > 0

    @property
    def _cp(self):
        """PeerComm address for the fused all-reduce of the current step, or None (single GPU, or a
        step shape the fused epilogue does not cover - those use NCCL, see ``_reduce``)."""
        return self.comm.ptr if (self.comm is not None and self._fused) else None

    def enable_dcp(self, dcp):
        """Shard the latent KV cache by token position over the tensor-parallel ranks (``dcp``: a ``parallel.dcp.DcpAttention`` for
        this model's heads).  Every rank then stores only its own tokens; the engine allocates pages for the local share.  The DSA
        indexer's key cache (its rows are 128-byte class, addressed by global position) stays replicated with a page table of its own.
        Call before the engine allocates the caches."""
        if dcp.world != self.tp_size or dcp.H != self.Hh * self.tp_size or dcp.dl != self.cfg.kv_lora or dcp.dr != self.cfg.qk_rope:
            raise ValueError("DcpAttention does not match this model's heads / latent sizes / ranks")
        self.dcp = dcp

    def _reduce(self, ws, R):
        """Row-parallel partial -> full sum when the fused in-kernel path is not in use."""
        if self.tp_size > 1 and not self._fused:
            import torch.distributed as dist
            dist.all_reduce(ws.sub[:R])

    def owns_expert(self, layer: int, e: int) -> bool:
        if self.expert_shard == "tp":
            return True                      # a slice of every expert
        if e < self.cfg.n_routed:
            return e % self.tp_size == self.tp_rank
        return layer % self.tp_size == self.tp_rank

    # ------------------------------------------------------------------ construction
    def _expert_lin(self, w, name: str, eq: str) -> QLinear:
        """One expert matrix in the arena's storage format.  Q4_K tensors of a GGUF checkpoint are taken as they are (bit-exact
        super-blocks); everything else goes through the float path (de-quantise, quantise to the arena format)."""
        if eq in GGML_OF and hasattr(w, "native_ggml"):
            nv = w.native_ggml(name)
            if nv is not None and nv[0] == GGML_OF[eq]:
                return QLinear.from_ggml(nv[0], nv[1], nv[2], nv[3], self.device)
        return QLinear.from_float(w[name], eq, self.device)

    def _gguf_layer_formats(self, w, prefix: str, e0: int):
        """(gate / up format, down format) when expert ``e0`` of this layer is stored in block types the kernels read natively
        (gate and up in the same type), else None."""
        if not hasattr(w, "native_ggml") or self.cfg.hidden % 256 or self.Fe % 256 or self.expert_shard == "tp":
            return None
        from ..formats import gguf as _gguf
        nm = prefix + (f"experts.{e0}." if e0 < self.cfg.n_routed else f"shared.{e0 - self.cfg.n_routed}.")
        ts = [w.native_ggml(nm + t) for t in ("gate", "up", "down")]
        if any(t is None for t in ts) or ts[0][0] != ts[1][0]:
            return None
        return _gguf.DEVICE_NATIVE[ts[0][0]], _gguf.DEVICE_NATIVE[ts[2][0]]

    def _lin(self, get, name, fmt):
        return QLinear.from_float(get(name), fmt, self.device)

    @classmethod
    def from_state_dict(cls, cfg: ModelConfig, w: Dict[str, torch.Tensor], device="cuda", kv_fmt="fp8", page=64,
                        expert_quant: Optional[str] = None, dense_quant: Optional[str] = None, tp_rank: int = 0,
                        tp_size: int = 1, expert_shard: Optional[str] = None, with_mtp: bool = False, layer_hook=None, skip_experts=None) -> "DeviceModel":
        """``skip_experts(i) -> bool``: leave MoE layer ``i``'s expert arena unbuilt (``L["arena"] = None``) - the layer hook provides it
        (an ``ExpertStreamer`` with a live GGUF source fills its pinned store from the file and creates the capped arena).
        ``layer_hook(i, L)``: called after layer ``i`` of the main stack is built (``ExpertStreamer.add_layer`` moves the layer's
        experts to pinned host memory there, so a model larger than HBM loads layer by layer).
        ``with_mtp``: also load the checkpoint's multi-token-prediction blocks (one more decoder layer each, with its experts)
        for ``forward_mtp`` / ``Engine.enable_mtp``; ignored where ``mtp_supported()`` is false or the checkpoint has none."""
        m = cls(cfg, device, kv_fmt, page, tp_rank, tp_size, expert_shard)
        dev = m.device
        tr, ts = tp_rank, tp_size

        def rows(t, n_units, unit):     # this rank's block of `n_units/ts` units of `unit` rows
            per = n_units // ts * unit
            return t[tr * per: (tr + 1) * per]

        def cols(t, n_units, unit):
            per = n_units // ts * unit
            return t[:, tr * per: (tr + 1) * per]
        eq = expert_quant or cfg.expert_quant
        dq = dense_quant or cfg.dense_quant
        gguf_experts = eq == "gguf"
        if eq.startswith("gguf"):
            # GGUF expert tensors: "gguf" = per layer the block types of the file where the kernels read them natively (Q4_K, Q5_K,
            # Q6_K, Q8_0, the down matrix possibly in another type than gate / up), else Q4_K; a named type = that type for all
            ok = cfg.hidden % 256 == 0 and m.Fe % 256 == 0 and m.expert_shard != "tp"
            eq = ("gguf_q4_k" if eq == "gguf" else eq) if ok else "bf16"
            if eq not in EXPERT_FMT or (eq == "gguf_q5_k" and not hasattr(w, "native_ggml")):
                eq = "gguf_q4_k"                    # types without a GPU decoder, or without a quantiser from float weights
        f32 = lambda t: t.to(dev).float().contiguous()
        m.embed = w["embed.weight"].to(dev).to(torch.bfloat16).contiguous()
        m.head = QLinear.from_float(rows(w["head.weight"], cfg.vocab, 1), "bf16", dev)
        m.final_norm = f32(w["final_norm.weight"])
        # multi-token-prediction blocks (layer ids n_layers ..): built like an MLA layer without indexer plus the block's input norms,
        # its [embedding ; stream] projection and its output norm.  Device path: one GPU, plain residual stream, FP8 / bf16 KV.
        n_mtp = cfg.n_mtp if (with_mtp and m.mtp_supported() and f"layers.{cfg.n_layers}.mtp.eh_proj" in w) else 0
        for i in range(cfg.n_layers + n_mtp):
            p = f"layers.{i}."
            is_mtp = i >= cfg.n_layers
            L: dict = {"attn_norm": f32(w[p + "attn_norm.weight"]), "ffn_norm": f32(w[p + "ffn_norm.weight"])}
            if is_mtp:
                L["mtp_enorm"], L["mtp_hnorm"] = f32(w[p + "mtp.enorm"]), f32(w[p + "mtp.hnorm"])
                L["mtp_eh"] = QLinear.from_float(w[p + "mtp.eh_proj"], "bf16", dev)
                L["mtp_final_norm"] = f32(w[p + "mtp.final_norm"])
            if cfg.mhc and not is_mtp:
                for nm in ("hc_attn", "hc_ffn"):
                    L[nm] = (f32(w[p + nm + ".fn"]), f32(w[p + nm + ".scale"]), f32(w[p + nm + ".base"]))
            if cfg.is_kda_layer(i):
                k = p + "kda."
                Hk, D = cfg.kda_heads, cfg.kda_head_dim
                L["kda_in"] = QLinear.from_float(torch.cat([rows(w[k + "q"], Hk, D), rows(w[k + "k"], Hk, D), rows(w[k + "v"], Hk, D),
                                                            rows(w[k + "beta"], Hk, 1), w[k + "f_a"], w[k + "g_a"]], 0), dq, dev)
                L["kda_fb"] = rows(w[k + "f_b"], Hk, D).to(dev).to(torch.bfloat16).contiguous()
                L["kda_gb"] = rows(w[k + "g_b"], Hk, D).to(dev).to(torch.bfloat16).contiguous()
                for nm in ("conv_q", "conv_k", "conv_v"):
                    L["kda_" + nm] = f32(rows(w[k + nm], Hk, D))
                L["kda_dt_bias"] = f32(rows(w[k + "dt_bias"], Hk, 1))
                L["kda_o_norm"] = f32(w[k + "o_norm"])
                L["kda_a_exp"] = torch.exp(f32(rows(w[k + "a_log"], Hk, 1)))
                L["kda_o"] = QLinear.from_float(cols(w[k + "o"], Hk, D), dq, dev)
            else:
                a = p + "attn."
                parts = [w[a + "q_a"], w[a + "kv_a"]]
                qb_parts = [rows(w[a + "q_b"], cfg.n_heads, cfg.qk_head)]
                has_idx = cfg.has_indexer and not is_mtp and cfg.index_source_layer(i) == i
                if has_idx:
                    x = p + "indexer."
                    parts += [w[x + "wk"], w[x + "weights_proj"]]
                    if cfg.index_kpool > 1:
                        parts.append(w[x + "gate"])
                        L["idx_ape"] = f32(w[x + "ape"])
                    qb_parts.append(w[x + "wq_b"])
                    L["idx_ln_w"] = f32(w[x + "k_norm.weight"]); L["idx_ln_b"] = f32(w[x + "k_norm.bias"])
                L["mla_in"] = QLinear.from_float(torch.cat(parts, 0), dq, dev)
                L["mla_qb"] = QLinear.from_float(torch.cat(qb_parts, 0), dq, dev)
                L["qa_norm"] = f32(w[a + "q_a_norm"]); L["kv_norm"] = f32(w[a + "kv_a_norm"])
                L["k_b"] = rows(w[a + "k_b"], cfg.n_heads, 1).to(dev).to(torch.bfloat16).contiguous()
                L["v_b"] = rows(w[a + "v_b"], cfg.n_heads, 1).to(dev).to(torch.bfloat16).contiguous()
                L["mla_o"] = QLinear.from_float(cols(w[a + "o"], cfg.n_heads, cfg.v_head), dq, dev)
            if cfg.is_moe_layer(i):
                mo = p + "moe."
                L["router"] = QLinear.from_float(w[mo + "router"], "f32", dev)
                L["router_bias"] = f32(w[mo + "router_bias"]) if (mo + "router_bias") in w else None
                if cfg.is_hash_layer(i):
                    L["tid2eid"] = w[mo + "tid2eid"].to(dev).to(torch.int32).contiguous()     # [vocab, top_k]
                E_total = cfg.n_routed + cfg.n_shared
                if skip_experts is not None and not is_mtp and ts == 1 and skip_experts(i):
                    L["arena"] = None                     # provided by the layer hook
                    m.layers.append(L)
                    if layer_hook is not None:
                        layer_hook(i, L)
                    if L["arena"] is None:
                        raise RuntimeError(f"layer {i}: the layer hook did not provide the expert arena it asked to skip")
                    continue
                mine = [e for e in range(E_total) if m.owns_expert(i, e)]
                eq_l, eq_dn = eq, eq
                if gguf_experts and mine:
                    # a GGUF checkpoint: this layer's experts in the block types of the file when the kernels read them natively
                    # (every expert of a layer shares its tensors' types; the shared expert may differ and is then converted)
                    nf = m._gguf_layer_formats(w, mo, mine[0])
                    if nf is not None:
                        eq_l, eq_dn = nf
                ef = expert_layout(eq_l, cfg.hidden, m.Fe, eq_dn)
                arena = ExpertArena(ef, max(len(mine), 1), E_total, dev)
                for s_, e in enumerate(mine):
                    nm = mo + (f"experts.{e}." if e < cfg.n_routed else f"shared.{e - cfg.n_routed}.")
                    if m.expert_shard == "tp":
                        # this GPU's slice of the expert: rows of gate / up, columns of down
                        f0, f1 = tr * m.Fe, (tr + 1) * m.Fe
                        parts = (QLinear.from_float(w[nm + "gate"][f0:f1], eq, dev), QLinear.from_float(w[nm + "up"][f0:f1], eq, dev),
                                 QLinear.from_float(w[nm + "down"][:, f0:f1].contiguous(), eq, dev))
                        arena.write_expert(s_, *parts)
                    else:
                        arena.write_expert(s_, m._expert_lin(w, nm + "gate", eq_l), m._expert_lin(w, nm + "up", eq_l), m._expert_lin(w, nm + "down", eq_dn))
                    arena.slot_of[e] = s_
                L["arena"] = arena
            else:
                f = p + "mlp."
                L["mlp_gu"] = QLinear.from_float(torch.cat([rows(w[f + "gate"], cfg.dense_inter, 1), rows(w[f + "up"], cfg.dense_inter, 1)], 0), dq, dev)
                L["mlp_down"] = QLinear.from_float(cols(w[f + "down"], cfg.dense_inter, 1), dq, dev)
            (m.mtp_layers if is_mtp else m.layers).append(L)
            if layer_hook is not None and not is_mtp:
                layer_hook(i, L)
        m._finish()
        return m

    @classmethod
    def random_init(cls, cfg: ModelConfig, device="cuda", kv_fmt="fp8", page=64, seed=0, expert_slots=None,
                    embed_on_host: bool = False, reserve_bytes: int = 4 << 30, tp_rank: int = 0, tp_size: int = 1,
                    expert_shard: Optional[str] = None, with_mtp: bool = False, layer_hook=None) -> "DeviceModel":
        """Random weights generated directly in storage format on the device (full-size models).
        ``layer_hook(i, L)``: called after the expert arena of MoE layer ``i`` is filled (``ExpertStreamer.add_layer``: every arena is
        then built with ALL of this rank's experts and handed over, whatever ``expert_slots`` says).
        ``expert_slots`` caps the routed-expert slots per MoE layer (VRAM expert cache): an int, None
        (all experts resident) or "auto" (as many as fit while leaving ``reserve_bytes`` of device
        memory free for caches and workspaces).  The first slots hold the shared experts followed by
        routed experts 0..; the rest start non-resident."""
        m = cls(cfg, device, kv_fmt, page, tp_rank, tp_size, expert_shard)
        dev = m.device
        gen = torch.Generator(device=dev).manual_seed(seed)                          # replicated tensors: same on every rank
        gloc = torch.Generator(device=dev).manual_seed(seed * 7919 + 1 + tp_rank)    # this rank's shards
        dq, eq = cfg.dense_quant, cfg.expert_quant
        if eq.startswith("gguf"):
            eq = "gguf_q4_k" if (cfg.hidden % 256 == 0 and m.Fe % 256 == 0) else "nvfp4"
        H = cfg.hidden

        def nrm(n):
            t = torch.empty(n, dtype=torch.float32, device=dev)
            t.normal_(1.0, 0.05, generator=gen)
            return t

        def rnd(*shape, std=0.02, dtype=torch.float32):
            t = torch.empty(*shape, dtype=dtype, device=dev)
            t.normal_(0.0, std, generator=gen)
            return t

        if embed_on_host:
            hg = torch.Generator().manual_seed(seed)
            e = torch.empty(cfg.vocab, H, dtype=torch.bfloat16).normal_(0.0, 1.0, generator=hg).pin_memory()
            m.embed = e
        else:
            m.embed = rnd(cfg.vocab, H, std=1.0, dtype=torch.bfloat16)
        m.head = QLinear.random(m.V_local, H, "bf16", dev, gen=gloc)

        def overwrite_rows(lin: QLinear, r0: int, std: float):
            """Re-draw rows [r0:] from the replicated generator (projections every rank must agree on)."""
            if lin.fmt == "bf16" and r0 < lin.N:
                lin.w[r0:].normal_(0.0, std, generator=gen)
        m.final_norm = nrm(H)
        n = cfg.hc_mult
        n_mtp = cfg.n_mtp if (with_mtp and m.mtp_supported()) else 0
        for i in range(cfg.n_layers + n_mtp):
            is_mtp = i >= cfg.n_layers                # a multi-token-prediction block: an MLA layer without indexer + its own norms / projection
            L: dict = {"attn_norm": nrm(H), "ffn_norm": nrm(H)}
            if is_mtp:
                L["mtp_enorm"], L["mtp_hnorm"], L["mtp_final_norm"] = nrm(H), nrm(H), nrm(H)
                L["mtp_eh"] = QLinear.random(H, 2 * H, "bf16", dev, std=0.05, gen=gen)
            if cfg.mhc and not is_mtp:
                for nm in ("hc_attn", "hc_ffn"):
                    L[nm] = (rnd(2 * n + n * n, n * H, std=0.05), torch.ones(3, device=dev), rnd(2 * n + n * n, std=0.5))
            if cfg.is_kda_layer(i):
                C = m.Hk * cfg.kda_head_dim
                L["kda_in"] = QLinear.random(3 * C + m.Hk + 2 * cfg.kda_rank, H, dq, dev, std=0.05, gen=gloc)
                overwrite_rows(L["kda_in"], 3 * C + m.Hk, 0.05)
                L["kda_fb"] = torch.empty(C, cfg.kda_rank, dtype=torch.bfloat16, device=dev).normal_(0.0, 0.2, generator=gloc)
                L["kda_gb"] = torch.empty(C, cfg.kda_rank, dtype=torch.bfloat16, device=dev).normal_(0.0, 0.2, generator=gloc)
                for nm in ("conv_q", "conv_k", "conv_v"):
                    L["kda_" + nm] = torch.empty(C, cfg.kda_conv, device=dev).uniform_(-0.5, 0.5, generator=gloc)
                L["kda_dt_bias"] = torch.empty(m.Hk, cfg.kda_head_dim, device=dev).uniform_(-1, 1, generator=gloc)
                L["kda_o_norm"] = nrm(cfg.kda_head_dim)
                L["kda_a_exp"] = torch.exp(torch.empty(m.Hk, device=dev).uniform_(-1.0, 1.5, generator=gloc))
                L["kda_o"] = QLinear.random(H, C, dq, dev, gen=gloc)
            else:
                Hh = m.Hh
                has_idx = cfg.has_indexer and not is_mtp and cfg.index_source_layer(i) == i
                n_in = cfg.q_lora + cfg.kv_lora + cfg.qk_rope
                n_qb = Hh * cfg.qk_head
                if has_idx:
                    n_in += cfg.index_head_dim + cfg.index_n_heads + (cfg.index_head_dim if cfg.index_kpool > 1 else 0)
                    n_qb += cfg.index_n_heads * cfg.index_head_dim
                    if cfg.index_kpool > 1:
                        L["idx_ape"] = rnd(cfg.index_kpool, cfg.index_head_dim, std=0.5)
                    L["idx_ln_w"] = nrm(cfg.index_head_dim); L["idx_ln_b"] = rnd(cfg.index_head_dim, std=0.1)
                L["mla_in"] = QLinear.random(_align(n_in, 8), H, dq, dev, std=0.05, gen=gen)
                L["mla_qb"] = QLinear.random(n_qb, cfg.q_lora, dq, dev, std=0.05, gen=gloc)
                overwrite_rows(L["mla_qb"], Hh * cfg.qk_head, 0.05)
                L["qa_norm"] = nrm(cfg.q_lora); L["kv_norm"] = nrm(cfg.kv_lora)
                L["k_b"] = torch.empty(Hh, cfg.kv_lora, cfg.qk_nope, dtype=torch.bfloat16, device=dev).normal_(0.0, 0.05, generator=gloc)
                L["v_b"] = torch.empty(Hh, cfg.v_head, cfg.kv_lora, dtype=torch.bfloat16, device=dev).normal_(0.0, 0.05, generator=gloc)
                L["mla_o"] = QLinear.random(H, Hh * cfg.v_head, dq, dev, gen=gloc)
            if cfg.is_moe_layer(i):
                L["router"] = QLinear.random(cfg.n_routed, H, "f32", dev, std=0.1, gen=gen)
                L["router_bias"] = rnd(cfg.n_routed, std=0.05) if cfg.router_bias else None
                if cfg.is_hash_layer(i):
                    # top_k distinct experts per token id: the first top_k columns of a row-wise random ranking
                    L["tid2eid"] = torch.rand(cfg.vocab, cfg.n_routed, device=dev, generator=gen).argsort(dim=1)[:, :cfg.top_k].to(torch.int32).contiguous()
                L["arena"] = None      # allocated below, once the non-expert footprint is known
            else:
                L["mlp_gu"] = QLinear.random(2 * m.Fd, H, dq, dev, gen=gloc)
                L["mlp_down"] = QLinear.random(H, m.Fd, dq, dev, gen=gloc)
            (m.mtp_layers if is_mtp else m.layers).append(L)
        moe_layers = [(i, L) for i, L in enumerate(m.layers + m.mtp_layers) if "arena" in L]
        if moe_layers:
            ef = expert_layout(eq, H, m.Fe)
            E_total = cfg.n_routed + cfg.n_shared
            max_owned = max(sum(1 for e in range(E_total) if m.owns_expert(i, e)) for i, _ in moe_layers)
            if expert_slots == "auto":
                free_b, _ = torch.cuda.mem_get_info(dev)
                free_b += torch.cuda.memory_reserved(dev) - torch.cuda.memory_allocated(dev)
                fit = int((free_b - reserve_bytes) // (ef.stride * len(moe_layers)))
                n_slots = max((cfg.top_k if m.expert_shard == "tp" else cfg.top_k // tp_size) + cfg.n_shared, min(max_owned, fit))
            elif expert_slots is None:
                n_slots = max_owned
            else:
                n_slots = min(max_owned, int(expert_slots) + cfg.n_shared)
            if layer_hook is not None:
                n_slots = max_owned
            m.expert_slots = n_slots
            for i, L in moe_layers:
                # resident order: this rank's shared expert first, then its routed experts by id
                order = [e for e in range(cfg.n_routed, E_total) if m.owns_expert(i, e)] + [e for e in range(cfg.n_routed) if m.owns_expert(i, e)]
                so = torch.full((E_total,), -1, dtype=torch.int32)
                for s_, e in enumerate(order[:n_slots]):
                    so[e] = s_
                arena = ExpertArena(ef, n_slots, E_total, dev)
                m._random_fill_arena(arena, eq, gloc)
                arena.slot_of.copy_(so)
                L["arena"] = arena
                if layer_hook is not None and i < cfg.n_layers:
                    layer_hook(i, L)
        m._finish()
        return m

    def _random_fill_arena(self, arena: ExpertArena, eq: str, gen):
        ef, d = arena.ef, arena.data
        if eq == "bf16":
            d.view(torch.bfloat16).normal_(0.0, 0.02, generator=gen)
        elif eq == "fp8_e4m3":
            d[:, : ef.off_sg].random_(0, 256, generator=gen)
            d[:, : ef.off_sg] &= 0xBF
            d[:, ef.off_sg: ef.off_tail].view(torch.float32).fill_(2.0 ** -5)        # a power of two next to 0.02 / 0.6
        elif eq == "gguf_q4_k":
            blocks = d[:, : ef.off_tail].view(d.shape[0], -1, 144)
            blocks.random_(0, 256, generator=gen)
            c = 0.02 * 3 ** 0.5
            blocks[:, :, :4] = torch.tensor([c / 7.5 / 24.0, c / 24.0], dtype=torch.float16).view(torch.uint8).to(d.device)
            blocks[:, :, 4:16] = (blocks[:, :, 4:16] & 0x0F) | 0x10
        else:
            d[:, : ef.off_sg].random_(0, 256, generator=gen)
            d[:, ef.off_sg: ef.off_tail].random_(0x30, 0x40, generator=gen)
            d[:, ef.off_tail: ef.off_tail + 12].view(torch.float32).fill_(0.02 / 2.1)

    def _fold_turboquant(self):
        """4-bit KV: attention runs in a rotated latent space.  The per-layer rotation is folded into W_UK / W_UV here, so
        the only run-time cost is the rotation of each new latent row when it is appended."""
        from ..formats import turboquant as tq
        cfg = self.cfg
        self.tq_centroids = tq.lloyd_max_gaussian(16).to(self.device)
        for i, L in enumerate(self.layers):
            if "k_b" not in L or "tq_rot_t" in L:
                continue
            rot = tq.rotation(cfg.kv_lora, i).to(self.device)
            L["k_b_orig"], L["v_b_orig"] = L["k_b"], L["v_b"]
            L["k_b"] = torch.einsum("ij,hjn->hin", rot, L["k_b"].float()).to(torch.bfloat16).contiguous()      # Pi @ W_UK[h]
            L["v_b"] = torch.einsum("hdl,il->hdi", L["v_b"].float(), rot).to(torch.bfloat16).contiguous()      # W_UV[h] @ Pi^T
            L["tq_rot_t"] = rot.T.contiguous().to(torch.bfloat16)

    def _finish(self):
        cfg = self.cfg
        for L in self.layers:
            if "kda_fb" in L and "kda_fb2" not in L:
                # [W | W]: the many-row KDA path computes the low-rank gates on the tensor cores with bf16 (hi | lo) activations
                L["kda_fb2"] = torch.cat([L["kda_fb"], L["kda_fb"]], 1).contiguous()
                L["kda_gb2"] = torch.cat([L["kda_gb"], L["kda_gb"]], 1).contiguous()
        if self.kv_fmt == "tq4":
            self._fold_turboquant()
        for L in self.layers + self.mtp_layers:
            if "kda_in" in L:
                self.max_proj = max(self.max_proj, L["kda_in"].N)
            if "mla_in" in L:
                self.max_proj = max(self.max_proj, L["mla_in"].N)
                self.max_qb = max(self.max_qb, L["mla_qb"].N)
        self._ef_bytes = {}

    def weight_bytes(self) -> int:
        tot = self.head.nbytes() + (self.embed.numel() * 2 if self.embed.is_cuda else 0)
        for L in self.layers + self.mtp_layers:
            for v in L.values():
                if isinstance(v, QLinear):
                    tot += v.nbytes()
                elif isinstance(v, ExpertArena):
                    tot += v.data.numel()
                elif isinstance(v, torch.Tensor):
                    tot += v.numel() * v.element_size()
                elif isinstance(v, tuple):
                    tot += sum(t.numel() * t.element_size() for t in v)
        return tot

    # ------------------------------------------------------------------ caches
    def alloc_cache(self, num_pages: int, n_slots: int, max_pages_per_seq: int):
        cfg, dev = self.cfg, self.device
        self.num_pages, self.n_slots, self.max_pages = num_pages, n_slots, max_pages_per_seq
        self.block_table = torch.zeros(n_slots, max_pages_per_seq, dtype=torch.int32, device=dev)
        # the indexer's key cache is addressed by GLOBAL position: with a sharded KV cache it stays replicated and gets its own
        # identity page table (slot-major, full length per slot); otherwise it shares the sequence's pages
        self.idx_block_table = self.block_table
        idx_pages = num_pages
        if (self.dcp is not None or self.idx_identity) and cfg.has_indexer:
            idx_pages = n_slots * max_pages_per_seq
            self.idx_block_table = torch.arange(idx_pages, dtype=torch.int32, device=dev).view(n_slots, max_pages_per_seq).contiguous()
        P = cfg.index_kpool
        for i in range(cfg.n_layers):
            if cfg.is_kda_layer(i):
                self.kda_state[i] = torch.zeros(n_slots, self.Hk, cfg.kda_head_dim, cfg.kda_head_dim, dtype=torch.float32, device=dev)
                self.kda_conv[i] = torch.zeros(n_slots, 3, self.Hk * cfg.kda_head_dim, 3, dtype=torch.float32, device=dev)
            else:
                self.kv_cache[i] = torch.zeros(num_pages, self.page, self.kv_row_bytes, dtype=torch.uint8, device=dev)
                if cfg.has_indexer and cfg.index_source_layer(i) == i:
                    self.idx_cache[i] = torch.zeros(idx_pages, self.page // P, self.idx_row_bytes, dtype=torch.uint8, device=dev)
                    if P > 1:
                        self.idx_tail[i] = torch.zeros(n_slots, P, 2, cfg.index_head_dim, dtype=torch.bfloat16, device=dev)
        for k in range(len(self.mtp_layers)):
            # a multi-token-prediction block keeps its own latent cache over the same pages (same positions, same page table)
            self.kv_cache[cfg.n_layers + k] = torch.zeros(num_pages, self.page, self.kv_row_bytes, dtype=torch.uint8, device=dev)

    def reset_slot(self, slot: int):
        for t in self.kda_state.values():
            t[slot].zero_()
        for t in self.kda_conv.values():
            t[slot].zero_()

    def cache_bytes_per_token(self) -> int:
        cfg = self.cfg
        b = 0
        for i in cfg.mla_layers():
            b += self.kv_row_bytes
            if cfg.has_indexer and cfg.index_source_layer(i) == i:
                b += self.idx_row_bytes // cfg.index_kpool
        return b

    # ------------------------------------------------------------------ forward
    def _ffn(self, i: int, L: dict, ws: Workspace, R: int, routed: bool = False, defer_combine: bool = False):
        """FFN sublayer into ``ws.sub``.  ``routed``: ids / weights of this layer are already in the workspace.  ``defer_combine``: leave the
        weighted sum of the expert outputs to the next hyper-connection kernel (returns True when it did so)."""
        cfg = self.cfg
        if "arena" not in L:
            L["mlp_gu"](ws.gu, ws.x, R, ldo=2 * self.Fd)
            nat.call("lsb_swiglu", ws.act_d, ws.gu, R, self.Fd, cfg.swiglu_limit)
            L["mlp_down"](ws.sub, ws.act_d, R, comm=self._cp)
            self._reduce(ws, R)
            return
        arena: ExpertArena = L["arena"]
        S = ws.S
        sc = {"sigmoid": 0, "softmax": 1, "sqrtsoftplus": 2}[cfg.scoring]
        if routed:
            pass        # the hyper-connection kernel in front of this layer already projected and selected (ws.ids / ws.wts)
        elif "tid2eid" in L:
            # hash layer: the experts are the table row of the row's token id, the weights their (unbiased) scores
            L["router"](ws.logits_r, ws.x, R)
            nat.call("lsb_router_hash", ws.logits_r, L["tid2eid"], ws.tok, ws.ids, ws.wts, R, cfg.n_routed, cfg.top_k, cfg.vocab,
                     sc, int(cfg.norm_topk_prob), cfg.routed_scale, cfg.n_shared, cfg.n_routed)
        elif ROUTER_FUSED and R <= 8 and cfg.hidden % 16 == 0 and R * (2 * cfg.n_routed + 128) * 4 <= 48 * 1024:
            # decode-sized steps: projection and top-k in one launch (the last block selects)
            nat.call("lsb_router_fused", L["router"].w, ws.x, ws.logits_r, L["router_bias"], ws.ids, ws.wts, ws.router_done, R, cfg.hidden,
                     cfg.n_routed, cfg.top_k, cfg.n_group, cfg.topk_group, sc, int(cfg.norm_topk_prob), cfg.routed_scale, cfg.n_shared)
        else:
            L["router"](ws.logits_r, ws.x, R)
            nat.call("lsb_router_topk", ws.logits_r, L["router_bias"], ws.ids, ws.wts, R, cfg.n_routed, cfg.top_k, cfg.n_group,
                     cfg.topk_group, sc, int(cfg.norm_topk_prob), cfg.routed_scale, cfg.n_shared, cfg.n_routed)
        if self.streamer is not None:
            # capped expert cache: experts are brought in from pinned host memory in waves; every wave runs the
            # expert kernels over what is resident, the combine runs once at the end over all slots
            present = self.streamer.run_layer(self, i, arena, ws, R)
        else:
            self._moe_prepare(arena, ws, R)
            self._moe_experts(arena, ws, R, ws.miss if self.tp_size == 1 else None)
            present = arena.slot_of
        if defer_combine and self.streamer is None and self._cp is None and self.tp_size == 1:
            return True
        nat.call("lsb_moe_combine", ws.sub, ws.y, ws.wts, ws.ids, present, R, S, cfg.hidden, 0, self._cp)
        if self.streamer is not None and self.streamer.cpu_partial is not None:
            ws.sub[:R].add_(self.streamer.cpu_partial)           # the experts the host computed for this step (capped cache, CPU offload)
        self._reduce(ws, R)
        return False

    def _moe_mode(self, arena: ExpertArena, ws: Workspace, R: int) -> str:
        cfg = self.cfg
        if getattr(ws, "tc_ok", False) and R >= TC_MOE_MIN_ROWS and arena.ef.fmt <= 3 and not arena.ef.fmt_down1:
            return "tc"
        fast_fp4 = arena.ef.fmt == 2 and self.Fe % 128 == 0 and cfg.hidden % 128 == 0
        return "pairs" if (fast_fp4 and R * ws.S <= 72) else "groups"

    def _moe_prepare(self, arena: ExpertArena, ws: Workspace, R: int):
        """Group the step's (row, slot) pairs by expert (once per layer, independent of residency)."""
        cfg, S = self.cfg, ws.S
        E_total = cfg.n_routed + cfg.n_shared
        mode = self._moe_mode(arena, ws, R)
        if mode == "tc":
            P = R * S
            nat.call("lsb_moe_tc_sort", ws.ids, P, E_total, ws.tc_bn, ws.tc_sorted, ws.tc_tile_e, ws.tc_tile_r0, ws.tc_tile_n, ws.tc_cnt)
            if ws.bs_ok:
                nat.call("lsb_quant_fp8_tiles" if ws.bs_fp8 else "lsb_quant_nvfp4_tiles", ws.x, 0, ws.tc_sorted, ws.tc_tile_r0, ws.tc_tile_n, ws.tc_cnt,
                         S, cfg.hidden, ws.tc_bn, min(ws.tc_tiles, P // ws.tc_bn + E_total + 1), ws.bs_xq, ws.bs_xsf, ws.bs_xa)
            else:
                nat.call("lsb_moe_tc_gather", ws.x, ws.tc_sorted, ws.tc_cnt, ws.tc_xs, P, S, cfg.hidden)
        elif mode == "groups":
            nat.call("lsb_moe_build_groups", ws.ids, R * S, E_total, ws.group_expert, ws.group_n, ws.group_pairs, ws.n_groups, ws.counts)

    def _moe_experts(self, arena: ExpertArena, ws: Workspace, R: int, miss):
        """gate/up + SwiGLU and down projections of every pair whose expert is resident (``arena.slot_of[e] >= 0``)."""
        cfg, S = self.cfg, ws.S
        E_total = cfg.n_routed + cfg.n_shared
        efp = ctypes.addressof(arena.ef)
        mode = self._moe_mode(arena, ws, R)
        if mode == "tc":
            P = R * S
            err = TcScratch.get(self.device).err
            tiles = min(ws.tc_tiles, P // ws.tc_bn + E_total + 1)
            if ws.bs_ok and ws.bs_fp8:
                wsf, og, ou, od = arena.bs_scale_atoms()
                a = (arena.data, arena.slot_of, efp, wsf, wsf.shape[1], og, ou, od, ws.tc_tile_e, ws.tc_tile_r0, ws.tc_tile_n, ws.tc_cnt, ws.tc_sorted)
                nat.call("lsb_moe_bs_ffn_fp8", 1, ws.bs_xq, ws.bs_xsf, ws.bs_xa, *a, ws.bs_act, ws.tc_bn, tiles, cfg.swiglu_limit, miss, err)
                nat.call("lsb_quant_fp8_tiles", ws.bs_act, 1, None, ws.tc_tile_r0, ws.tc_tile_n, ws.tc_cnt, S, self.Fe, ws.tc_bn, tiles,
                         ws.bs_aq, ws.bs_asf, ws.bs_aa)
                nat.call("lsb_moe_bs_ffn_fp8", 0, ws.bs_aq, ws.bs_asf, ws.bs_aa, *a, ws.y, ws.tc_bn, tiles, 0.0, None, err)
                return
            if ws.bs_ok:
                a = (arena.data, arena.slot_of, efp, ws.tc_tile_e, ws.tc_tile_r0, ws.tc_tile_n, ws.tc_cnt, ws.tc_sorted)
                nat.call("lsb_moe_bs_ffn", 1, ws.bs_xq, ws.bs_xsf, ws.bs_xa, *a, ws.bs_act, ws.tc_bn, tiles, cfg.swiglu_limit, miss, err)
                nat.call("lsb_quant_nvfp4_tiles", ws.bs_act, 1, None, ws.tc_tile_r0, ws.tc_tile_n, ws.tc_cnt, S, self.Fe, ws.tc_bn, tiles,
                         ws.bs_aq, ws.bs_asf, ws.bs_aa)
                nat.call("lsb_moe_bs_ffn", 0, ws.bs_aq, ws.bs_asf, ws.bs_aa, *a, ws.y, ws.tc_bn, tiles, 0.0, None, err)
                return
            nat.call("lsb_moe_tc_ffn", 1, ws.tc_xs, ws.tc_xs.shape[0], arena.data, arena.slot_of, efp, ws.tc_tile_e, ws.tc_tile_r0, ws.tc_tile_n,
                     ws.tc_cnt, ws.tc_sorted, ws.tc_act, ws.tc_bn, tiles, cfg.swiglu_limit, miss, err, None)
            nat.call("lsb_moe_tc_ffn", 0, ws.tc_act, ws.tc_act.shape[0], arena.data, arena.slot_of, efp, ws.tc_tile_e, ws.tc_tile_r0, ws.tc_tile_n,
                     ws.tc_cnt, ws.tc_sorted, ws.y, ws.tc_bn, tiles, 0.0, None, err, None)
        elif mode == "pairs":
            # small batch: every (row, slot) pair streams its expert on its own - no grouping pass
            # blocks per expert: finer when this GPU holds only a share of the step's experts (expert parallel), see the kernels
            # (sliced experts keep every expert on every GPU with 1/N of the rows of gate / up and 1/N of the columns of down: the
            # down projection keeps its row count, so it keeps the widest block)
            run_gu = MOE_RUN_GU or (8 if self.tp_size == 1 else (4 if self.tp_size == 2 else 2))
            run_dn = MOE_RUN_DN or (16 if self.tp_size == 1 or self.expert_shard == "tp" else (8 if self.tp_size == 2 else 4))
            nat.call("lsb_moe_gateup", ws.x, arena.data, arena.slot_of, efp, ws.ids, None, None, None, ws.act, S, R * S, cfg.swiglu_limit, miss, run_gu)
            nat.call("lsb_moe_down", ws.act, arena.data, arena.slot_of, efp, ws.ids, None, None, None, ws.y, R * S, run_dn)
        else:
            mg = min(ws.max_groups, min(R * S, (R * S + 3) // 4 + E_total))
            nat.call("lsb_moe_gateup", ws.x, arena.data, arena.slot_of, efp, ws.group_expert, ws.group_n, ws.group_pairs, ws.n_groups,
                     ws.act, S, mg, cfg.swiglu_limit, miss, 0)
            nat.call("lsb_moe_down", ws.act, arena.data, arena.slot_of, efp, ws.group_expert, ws.group_n, ws.group_pairs, ws.n_groups,
                     ws.y, mg, 0)

    def _kda(self, i: int, L: dict, ws: Workspace, R: int, nseq: int):
        cfg = self.cfg
        C = self.Hk * cfg.kda_head_dim
        lin: QLinear = L["kda_in"]
        lin(ws.proj, ws.x, R, ldo=self.max_proj)
        args = (ws.proj, self.max_proj, 0, C, 2 * C, 3 * C, 3 * C + self.Hk,
                3 * C + self.Hk + cfg.kda_rank, cfg.kda_rank, L["kda_fb"], L["kda_gb"], L.get("kda_fb2"), L.get("kda_gb2"), L["kda_conv_q"], L["kda_conv_k"],
                L["kda_conv_v"], L["kda_a_exp"], L["kda_dt_bias"], L["kda_o_norm"], self.kda_state[i], self.kda_conv[i],
                ws.seq_row0, ws.seq_nrows, ws.seq_slot, ws.kda_out, nseq, self.Hk, cfg.kda_head_dim,
                cfg.kda_head_dim ** -0.5, cfg.kda_lower_bound, cfg.rms_eps, R, ws.kda_scratch)
        if ws.kda_chunk_ws is not None and nseq == 1 and R >= 128:
            nat.call("lsb_kda_forward_chunked", *args, ws.kda_chunk_ws, ws.kda_chunk_ws.numel())
        else:
            nat.call("lsb_kda_forward", *args)
        L["kda_o"](ws.sub, ws.kda_out, R, comm=self._cp)
        self._reduce(ws, R)

    def _mla(self, i: int, L: dict, ws: Workspace, R: int, dense: bool = False):
        """``dense``: the layer has no indexer and attends over the whole prefix (multi-token-prediction blocks)."""
        cfg = self.cfg
        Hh, dl, dr, dn, dv = self.Hh, cfg.kv_lora, cfg.qk_rope, cfg.qk_nope, cfg.v_head
        ldp = self.max_proj
        off_qa, off_kv = 0, cfg.q_lora
        off_ik = off_kv + dl + dr
        off_iw = off_ik + cfg.index_head_dim
        off_ig = off_iw + cfg.index_n_heads
        src = cfg.index_source_layer(i) if (cfg.has_indexer and not dense) else -1
        has_idx = src == i
        L["mla_in"](ws.proj, ws.x, R, ldo=ldp)
        P = cfg.index_kpool
        if has_idx:
            nat.call("lsb_indexer_k_append", ws.proj, ldp, off_ik, off_ig, L["idx_ln_w"], L["idx_ln_b"], L.get("idx_ape"),
                     self.inv_freq_idx, cfg.index_rope_dim, self.idx_cache[i], self.idx_block_table, self.max_pages, self.page // P,
                     self.idx_tail.get(i), ws.kstash, ws.row_seq, ws.row_pos, ws.row_slot, R, P, 1e-6)
        nat.call("lsb_mla_prep", ws.proj, ldp, off_qa, cfg.q_lora, off_kv, dl, dr, L["qa_norm"], L["kv_norm"], self.inv_freq,
                 ws.q_c, self.kv_cache[i], self.block_table, self.max_pages, ws.row_seq, ws.row_pos, R, self.page,
                 KV_FMT[self.kv_fmt], cfg.rms_eps, L.get("tq_rot_t"), self.tq_centroids, ws.row_store if self.dcp is not None else None)
        ldq = self.max_qb
        L["mla_qb"](ws.qproj, ws.q_c, R, ldo=ldq)
        nat.call("lsb_batched_gemv_bf16", ws.q_abs, ws.qproj, L["k_b"], R, Hh, dl, dn, ldq, dn + dr, Hh * (dl + dr), dl + dr,
                 dr, self.inv_freq, ws.row_pos)
        sel_idx = sel_cnt = None
        sel_ld = 0
        if cfg.has_indexer and not dense:
            if has_idx:
                nat.call("lsb_indexer_q_prep", ws.qproj, ldq, Hh * (dn + dr), ws.proj, ldp, off_iw, cfg.index_n_heads,
                         cfg.index_rope_dim, self.inv_freq_idx, ws.row_pos, ws.q_idx, ws.idx_w, ws.kstash, off_ig,
                         self.idx_tail.get(i), ws.row_seq, ws.row_slot, P, R)
                if getattr(ws, "idx_tc", False) and ws.single_seq and R >= 64 and 0 < ws.ne_hint <= ws.idx_kbf_rows:
                    # a prefill chunk: every row scores the same sequence's keys - one GEMM on the tensor cores
                    nat.call("lsb_indexer_score_tc", ws.q_idx, ws.idx_w, cfg.index_n_heads, self.idx_cache[i], self.idx_block_table,
                             self.max_pages, self.page // P, ws.row_seq, ws.n_entries, ws.scores, ws.max_entries, R, ws.ne_hint,
                             ws.idx_kbf, ws.idx_kbf_rows, ws.idx_kscale, TcScratch.get(self.device).err)
                elif getattr(ws, "idx_f8", False):
                    # few rows over a long index row: FP8 x FP8 on the tensor cores straight over the cached keys
                    nat.call("lsb_indexer_score_f8", ws.q_idx, ws.idx_w, cfg.index_n_heads, self.idx_cache[i], self.idx_cache[i].shape[0],
                             self.idx_block_table, self.max_pages, self.page // P, ws.row_seq, ws.n_entries, ws.scores, ws.max_entries, R,
                             ws.max_entries, TcScratch.get(self.device).err)
                else:
                    nat.call("lsb_indexer_score", ws.q_idx, ws.idx_w, cfg.index_n_heads, self.idx_cache[i], self.idx_block_table,
                             self.max_pages, self.page // P, ws.row_seq, ws.n_entries, ws.scores, ws.max_entries, R, ws.max_entries)
                if ws.topk_scratch is not None:
                    nat.call("lsb_indexer_topk_split", ws.scores, ws.max_entries, ws.n_entries, ws.row_len, ws.row_seq,
                             cfg.index_topk // P, P, ws.sel_idx, ws.sel_cnt, ws.sel_ld, R, ws.max_entries, ws.topk_scratch)
                else:
                    nat.call("lsb_indexer_topk", ws.scores, ws.max_entries, ws.n_entries, ws.row_len, ws.row_seq,
                             cfg.index_topk // P, P, ws.sel_idx, ws.sel_cnt, ws.sel_ld, R)
            sel_idx, sel_cnt, sel_ld = ws.sel_idx, ws.sel_cnt, ws.sel_ld
        if self.dcp is not None:
            # sharded KV: gather the queries of all heads, attend over this rank's token shard, merge on the head owners
            self.dcp.forward(ws.q_abs, self.kv_cache[i], self.block_table, self.max_pages, ws.row_seq, ws.row_len_local, ws.o_lat, self.page,
                             KV_FMT[self.kv_fmt], cfg.softmax_scale, sel_idx=sel_idx, sel_cnt=sel_cnt, tq_centroids=self.tq_centroids, rows=R)
        elif self.row_tier is not None and sel_idx is not None and self.row_tier.step_has_cold(R):
            # (a step none of whose sequences has a page in the cold tier - e.g. the prefill of a fresh prompt - reads the paged cache directly)
            # tiered KV: the selected rows (hot pages and cold tier alike) are materialised in a dense buffer, attention runs over that
            cache_m, bt_m, pm, seq_m, sel_m = self.row_tier.materialise(i, ws, R, sel_idx, sel_cnt, sel_ld)
            nat.call("lsb_mla_decode", ws.q_abs, cache_m, bt_m, pm, seq_m, sel_cnt, sel_m, sel_cnt, sel_ld, ws.o_lat, None, ws.o_part, ws.ml_part,
                     R, Hh, dl, dr, self.page, KV_FMT[self.kv_fmt], ws.NS, cfg.softmax_scale, self.tq_centroids)
        else:
            nat.call("lsb_mla_decode", ws.q_abs, self.kv_cache[i], self.block_table, self.max_pages, ws.row_seq, ws.row_len,
                     sel_idx, sel_cnt, sel_ld, ws.o_lat, None, ws.o_part, ws.ml_part, R, Hh, dl, dr, self.page,
                     KV_FMT[self.kv_fmt], ws.NS, cfg.softmax_scale, self.tq_centroids)
        nat.call("lsb_batched_gemv_bf16", ws.attn_v, ws.o_lat, L["v_b"], R, Hh, dv, dl, Hh * dl, dl, Hh * dv, dv, 0, None, None)
        L["mla_o"](ws.sub, ws.attn_v, R, comm=self._cp)
        self._reduce(ws, R)

    def _mhc_cluster_ok(self) -> bool:
        """Whether the one-launch cluster kernel covers this model's hyper-connection pass on this device (asked once)."""
        if not hasattr(self, "_mhc_clus"):
            self._mhc_clus = MHC_CLUSTER and nat.call("lsb_mhc_cluster_width", self.cfg.hidden, self.cfg.hc_mult) > 0
        return self._mhc_clus

    def _router_foldable(self, ws: "Workspace") -> bool:
        cfg = self.cfg
        return MHC_FOLD_ROUTER and cfg.n_routed <= 2048 and cfg.top_k <= 32 and cfg.n_group <= 64 and cfg.n_shared <= 32

    def _hc_pass(self, hc, norm_w, ws: "Workspace", R: int, mode: int, clus: bool, pending, route):
        """post of the previous sublayer + pre of the next one: residual streams, mixing gates, contracted and normalised input
        ``ws.x``.  ``pending``: slot table of a MoE layer whose expert outputs (``ws.y``) still have to be combined;
        ``route``: the MoE layer whose router runs on the new ``ws.x`` inside the same kernel."""
        cfg = self.cfg
        fn, sc, base = hc
        H, n = cfg.hidden, cfg.hc_mult
        if clus:
            S = getattr(ws, "S", 0)
            rs = {"sigmoid": 0, "softmax": 1, "sqrtsoftplus": 2}[cfg.scoring]
            nat.call("lsb_mhc_cluster", ws.x, ws.resid, ws.sub, ws.post, ws.comb, fn, sc, base, norm_w, R, H, n, mode, cfg.hc_sinkhorn_iters,
                     cfg.hc_eps, cfg.rms_eps, cfg.hc_post_mult,
                     ws.y if pending is not None else None, ws.wts if pending is not None else None, ws.ids if pending is not None else None,
                     pending, S,
                     route["router"].w if route is not None else None, route["router_bias"] if route is not None else None,
                     ws.logits_r if route is not None else None, ws.ids if route is not None else None, ws.wts if route is not None else None,
                     cfg.n_routed, cfg.top_k, cfg.n_group, cfg.topk_group, rs, int(cfg.norm_topk_prob), cfg.routed_scale, cfg.n_shared,
                     self._cp if pending is None else None)
            return
        assert pending is None and route is None
        nat.call("lsb_mhc_post_pre", ws.x, ws.resid, ws.sub, ws.post, ws.comb, fn, sc, base, norm_w, ws.part, R, H, n,
                 mode, cfg.hc_sinkhorn_iters, cfg.hc_eps, cfg.rms_eps, cfg.hc_post_mult, ws.hc_done, ws.hc_pre, self._cp)

    def set_aux_capture(self, layer_ids=(), rows: int = 0):
        """Keep, for every step from now on, the stream that ENTERS each layer of ``layer_ids`` (hyper-connection models: the mean over
        the residual streams; ``n_layers`` = the stream leaving the last layer, models without hyper-connections only) for the step's
        rows: ``aux_capture["buf"][:R].view(R, -1)`` is the concatenation in the order of ``layer_ids`` - the features a block draft
        model is conditioned on (``speculation/dspark.py``).  The copies are part of the step (and of its CUDA graph): the caller
        drops graphs captured before.  An empty ``layer_ids`` switches the capture off.
        Reference: the aux-hidden export hook in front of every layer's attention (src/daemon/dispatch_forward.cpp)."""
        ids = [int(l) for l in layer_ids]
        if not ids:
            self.aux_capture = None
            return
        n = self.cfg.n_layers
        if self.tp_size > 1:
            raise NotImplementedError("aux hidden capture is built for one GPU")
        if any(l < 0 or l > n or (l == n and self.cfg.mhc) for l in ids) or len(set(ids)) != len(ids):
            raise ValueError(f"aux layers {ids} do not fit a model of {n} layers" + (" with hyper-connections (no un-normalised final stream)" if self.cfg.mhc else ""))
        self.aux_capture = {"slots": {l: j for j, l in enumerate(ids)},
                            "buf": torch.zeros(max(1, int(rows)), len(ids), self.cfg.hidden, dtype=torch.bfloat16, device=self.device)}

    def _capture_aux(self, i: int, ws: Workspace, R: int):
        ac = self.aux_capture
        j = ac["slots"].get(i)
        if j is None:
            return
        if R > ac["buf"].shape[0]:
            raise RuntimeError(f"a step of {R} rows exceeds the aux capture buffer ({ac['buf'].shape[0]} rows)")
        H = self.cfg.hidden
        if self.cfg.mhc:
            ac["buf"][:R, j].copy_(ws.resid[:R].mean(1))
        else:
            ac["buf"][:R, j].copy_(ws.resid.view(-1)[: ws.R * H].view(ws.R, H)[:R])

    def set_layer_skip(self, skip=(), probe: bool = False):
        """Layer skipping for draft passes: ``skip`` = layers to leave out (the first and the last layer are never skipped), ``probe`` =
        record, per executed layer l, the cosine similarity between the normalised input of l and of the next executed layer (row 0 of
        the step) in ``self.probe["sims"][l]`` - "how much did layer l change its input".  Reference: layer skip during the
        self-speculative draft (python/orchestrator/layer_skip.py; src/compute/kernels/similarity/cosine_sim.h)."""
        n = self.cfg.n_layers
        self.skip_layers = frozenset(int(l) for l in skip if 0 < int(l) < n - 1)
        if probe and self.probe is None:
            self.probe = {"prev": torch.zeros(1, self.cfg.hidden, dtype=torch.bfloat16, device=self.device),
                          "sims": torch.zeros(n, dtype=torch.float32, device=self.device)}
        if not probe:
            self.probe = None

    def _probe_input(self, i: int, ws: Workspace, last: int) -> int:
        """Called when ``ws.x`` holds the input of layer i; ``last`` = the previously executed layer (-1 for none)."""
        pr = self.probe
        if pr is None:
            return i
        H = self.cfg.hidden
        if last >= 0:
            nat.call("lsb_cosine_sim", pr["prev"], ws.x, 1, H, H, H, pr["sims"][last: last + 1])
        pr["prev"].copy_(ws.x[:1])
        return i

    def forward(self, ws: Workspace, R: int, nseq: int, logit_row0: int, n_logit_rows: int):
        """Run one step over the first ``R`` rows of the workspace (inputs already staged in
        ``ws``).  Writes logits for rows [logit_row0, logit_row0 + n_logit_rows)."""
        cfg = self.cfg
        H, n = cfg.hidden, cfg.hc_mult
        # fused in-kernel all-reduce: GEMV epilogues cover 1, 2 or 4 rows; the tcgen05 GEMM epilogue covers any larger
        # step with bf16 dense weights, as long as the step fits the peers' receive slots
        # in-kernel NVLink all-reduce whenever the partial fits the peer buffers (fused GEMV / GEMM epilogues where they exist,
        # a push kernel after the layer otherwise); NCCL only beyond that
        self._fused = self.comm is not None and R * H <= self.comm.cap
        if self.comm is not None:
            # fewer than 8 rows: the kernel that consumes a cross-rank sum exchanges the partials itself (one flag per CTA) instead of
            # the producer's last block copying them to every peer; needs the cluster form of the hyper-connection pass where there is one
            xchg = COMM_XCHG if (self._fused and R < 8 and R <= MHC_CLUSTER_MAX_ROWS and self.dcp is None and (not cfg.mhc or self._mhc_cluster_ok())) else 0
            if xchg == 2 and R * H > self.comm.ll_cap:
                xchg = 1
            self.comm.struct.xchg = xchg
        if self.dcp is not None:
            nat.call("lsb_dcp_rows", ws.row_pos, ws.row_len, ws.row_store, ws.row_len_local, R, self.dcp.chunk, self.tp_size, self.tp_rank)
        if cfg.mhc:
            nat.call("lsb_embedding", ws.sub, None, self.embed, ws.tok, R, H, 0, cfg.vocab)
            # decode-sized steps: one cluster kernel per post -> pre pass, with the MoE combine folded in front and the router behind
            clus = R <= MHC_CLUSTER_MAX_ROWS and self._mhc_cluster_ok()
            pending = None         # slot table of the MoE layer whose combine the next pass performs
            last_run = -1
            for i, L in enumerate(self.layers):
                if i in self.skip_layers:
                    continue                 # the pending sublayer output, its gates and the residual streams wait for the next executed pass
                self._hc_pass(L["hc_attn"], L["attn_norm"], ws, R, 0 if i == 0 else 1, clus, pending, None)
                pending = None
                if self.aux_capture is not None:
                    self._capture_aux(i, ws, R)          # the residual streams now hold what enters layer i
                last_run = self._probe_input(i, ws, last_run)
                if cfg.is_kda_layer(i):
                    self._kda(i, L, ws, R, nseq)
                else:
                    self._mla(i, L, ws, R)
                route = L if (clus and "arena" in L and "tid2eid" not in L and self._router_foldable(ws)) else None
                self._hc_pass(L["hc_ffn"], L["ffn_norm"], ws, R, 1, clus, None, route)
                last = i + 1 == len(self.layers)
                if self._ffn(i, L, ws, R, routed=route is not None, defer_combine=MHC_FOLD_COMBINE and clus and not last and self.drift is None):
                    pending = L["arena"].slot_of
                if self.drift is not None:
                    self.drift[f"layer{i:03d}.ffn_out"] = ws.sub[:R].float().cpu()
            nat.call("lsb_mhc_contract_norm", ws.x, ws.resid, ws.sub, ws.post, ws.comb, self.final_norm, R, H, n, cfg.rms_eps, self._cp)
        else:
            resid = ws.resid.view(-1)[: ws.R * H].view(ws.R, H)
            nat.call("lsb_embedding", resid, None, self.embed, ws.tok, R, H, 0, cfg.vocab)
            nat.call("lsb_rmsnorm", ws.x, resid, self.layers[0]["attn_norm"], R, H, H, H, cfg.rms_eps, 1, None)
            last_run = -1
            for i, L in enumerate(self.layers):
                nxt = self.layers[i + 1]["attn_norm"] if i + 1 < cfg.n_layers else self.final_norm
                if self.aux_capture is not None:
                    self._capture_aux(i, ws, R)
                if i in self.skip_layers:
                    # the residual stays as it is; only the normalisation weights change to the next layer's
                    nat.call("lsb_rmsnorm", ws.x, resid, nxt, R, H, H, H, cfg.rms_eps, 1, None)
                    continue
                last_run = self._probe_input(i, ws, last_run)
                if cfg.is_kda_layer(i):
                    self._kda(i, L, ws, R, nseq)
                else:
                    self._mla(i, L, ws, R)
                nat.call("lsb_add_rmsnorm", ws.x, resid, ws.sub, L["ffn_norm"], R, H, cfg.rms_eps, self._cp)
                self._ffn(i, L, ws, R)
                nat.call("lsb_add_rmsnorm", ws.x, resid, ws.sub, nxt, R, H, cfg.rms_eps, self._cp)
                if self.drift is not None:
                    self.drift[f"layer{i:03d}.resid"] = resid[:R].float().cpu()
            if self.aux_capture is not None:
                self._capture_aux(cfg.n_layers, ws, R)
        xr = ws.x[logit_row0: logit_row0 + n_logit_rows]
        self.head(ws.logits, xr, n_logit_rows)
        if self.drift is not None:
            self.drift["final_norm_out"] = xr.float().cpu()
            self.drift["logits"] = ws.logits[:n_logit_rows].float().cpu()

    def forward_mtp(self, ws: Workspace, R: int, k: int = 0, logit_row0: int = 0, n_logit_rows: int = 0):
        """Multi-token-prediction block ``k`` over the staged rows.  In: ``ws.resid`` rows = the stream of the previous depth at the
        rows' positions (after ``forward``: the main model's stream in front of its output norm), ``ws.tok`` = the token one place
        AHEAD of each row's position, the rows' sequence / position arrays as staged for the main step.  Does
            x = eh_proj [RMSNorm_e(Emb(tok)) ; RMSNorm_h(stream)],  one decoder block (dense MLA over the block's own latent cache,
            FFN / MoE),  logits = head(RMSNorm_f(stream'))
        and leaves the block's output stream in ``ws.resid`` (the input of the next depth), logits of rows
        [logit_row0, logit_row0 + n_logit_rows) in ``ws.logits``.  Reference: the engine's MtpSpeculationMethod (src/speculation/),
        python/orchestrator/mtp_draft.py; architecture: DeepSeek-V3 technical report, section 2.2."""
        cfg = self.cfg
        if not self.mtp_layers:
            raise RuntimeError("this model has no multi-token-prediction blocks on the device")
        if self.streamer is not None or self.row_tier is not None:
            raise RuntimeError("multi-token-prediction blocks need resident experts and an untiered KV cache")
        L = self.mtp_layers[k]
        i = cfg.n_layers + k
        H = cfg.hidden
        self._fused = False
        resid = ws.resid.view(-1)[: ws.R * H].view(ws.R, H)
        cat = ws.mtp_cat
        nat.call("lsb_embedding", ws.sub, None, self.embed, ws.tok, R, H, 0, cfg.vocab)
        nat.call("lsb_rmsnorm", cat, ws.sub, L["mtp_enorm"], R, H, H, 2 * H, cfg.rms_eps, 1, None)
        nat.call("lsb_rmsnorm", cat.view(-1)[H:], resid, L["mtp_hnorm"], R, H, H, 2 * H, cfg.rms_eps, 1, None)
        L["mtp_eh"](resid, cat, R)                               # the block's residual stream replaces the previous depth's
        nat.call("lsb_rmsnorm", ws.x, resid, L["attn_norm"], R, H, H, H, cfg.rms_eps, 1, None)
        self._mla(i, L, ws, R, dense=True)
        nat.call("lsb_add_rmsnorm", ws.x, resid, ws.sub, L["ffn_norm"], R, H, cfg.rms_eps, None)
        self._ffn(i, L, ws, R)
        nat.call("lsb_add_rmsnorm", ws.x, resid, ws.sub, L["mtp_final_norm"], R, H, cfg.rms_eps, None)
        if n_logit_rows:
            self.head(ws.logits, ws.x[logit_row0: logit_row0 + n_logit_rows], n_logit_rows)

    def argmax(self, ws: Workspace, n_rows: int):
        """Greedy token per row; with a vocabulary-parallel head the per-rank winners are exchanged
        in-kernel over NVLink (8 bytes per row per rank)."""
        nat.call("lsb_argmax", ws.logits, self.V_local, n_rows, self.V_local, ws.amax_part, ws.out_tok, ws.out_val,
                 self.tp_rank * self.V_local, self.comm_amax.ptr if self.comm_amax is not None else None)

    # ------------------------------------------------------------------ oracle support
    def effective_state_dict(self) -> Dict[str, torch.Tensor]:
        """fp32 CPU state dict of what the device actually computes with (dequantised), in the
        canonical naming - lets the oracle check the kernels independent of quantisation error."""
        cfg = self.cfg
        out: Dict[str, torch.Tensor] = {}
        cpu = lambda t: t.detach().float().cpu()
        out["embed.weight"] = cpu(self.embed)
        out["head.weight"] = cpu(self.head.dequant())
        out["final_norm.weight"] = cpu(self.final_norm)
        for i, L in enumerate(self.layers + self.mtp_layers):
            p = f"layers.{i}."
            out[p + "attn_norm.weight"] = cpu(L["attn_norm"]); out[p + "ffn_norm.weight"] = cpu(L["ffn_norm"])
            if "mtp_eh" in L:
                out[p + "mtp.enorm"], out[p + "mtp.hnorm"], out[p + "mtp.final_norm"] = cpu(L["mtp_enorm"]), cpu(L["mtp_hnorm"]), cpu(L["mtp_final_norm"])
                out[p + "mtp.eh_proj"] = cpu(L["mtp_eh"].dequant())
            if cfg.mhc and "hc_attn" in L:
                for nm in ("hc_attn", "hc_ffn"):
                    out[p + nm + ".fn"], out[p + nm + ".scale"], out[p + nm + ".base"] = (cpu(t) for t in L[nm])
            if cfg.is_kda_layer(i):
                C = cfg.kda_heads * cfg.kda_head_dim
                w = cpu(L["kda_in"].dequant())
                k = p + "kda."
                out[k + "q"], out[k + "k"], out[k + "v"] = w[:C], w[C:2 * C], w[2 * C:3 * C]
                o = 3 * C
                out[k + "beta"] = w[o: o + cfg.kda_heads]; o += cfg.kda_heads
                out[k + "f_a"] = w[o: o + cfg.kda_rank]; o += cfg.kda_rank
                out[k + "g_a"] = w[o: o + cfg.kda_rank]
                out[k + "f_b"] = cpu(L["kda_fb"]); out[k + "g_b"] = cpu(L["kda_gb"])
                for nm in ("conv_q", "conv_k", "conv_v", "dt_bias", "o_norm"):
                    out[k + nm] = cpu(L["kda_" + nm])
                out[k + "a_log"] = torch.log(cpu(L["kda_a_exp"]))
                out[k + "o"] = cpu(L["kda_o"].dequant())
            else:
                a = p + "attn."
                w = cpu(L["mla_in"].dequant())
                out[a + "q_a"] = w[: cfg.q_lora]
                o = cfg.q_lora
                out[a + "kv_a"] = w[o: o + cfg.kv_lora + cfg.qk_rope]; o += cfg.kv_lora + cfg.qk_rope
                wq = cpu(L["mla_qb"].dequant())
                nq = cfg.n_heads * cfg.qk_head
                out[a + "q_b"] = wq[:nq]
                if cfg.has_indexer and i < cfg.n_layers and cfg.index_source_layer(i) == i:
                    x = p + "indexer."
                    out[x + "wk"] = w[o: o + cfg.index_head_dim]; o += cfg.index_head_dim
                    out[x + "weights_proj"] = w[o: o + cfg.index_n_heads]; o += cfg.index_n_heads
                    if cfg.index_kpool > 1:
                        out[x + "gate"] = w[o: o + cfg.index_head_dim]
                        out[x + "ape"] = cpu(L["idx_ape"])
                    out[x + "wq_b"] = wq[nq:]
                    out[x + "k_norm.weight"] = cpu(L["idx_ln_w"]); out[x + "k_norm.bias"] = cpu(L["idx_ln_b"])
                out[a + "q_a_norm"] = cpu(L["qa_norm"]); out[a + "kv_a_norm"] = cpu(L["kv_norm"])
                out[a + "k_b"] = cpu(L.get("k_b_orig", L["k_b"])); out[a + "v_b"] = cpu(L.get("v_b_orig", L["v_b"]))
                out[a + "o"] = cpu(L["mla_o"].dequant())
            if "arena" in L:
                mo = p + "moe."
                out[mo + "router"] = cpu(L["router"].w)
                if L["router_bias"] is not None:
                    out[mo + "router_bias"] = cpu(L["router_bias"])
                if "tid2eid" in L:
                    out[mo + "tid2eid"] = L["tid2eid"].cpu()
                arena: ExpertArena = L["arena"]
                fmt = {v: k for k, v in EXPERT_FMT.items()}[arena.ef.fmt]
                so = arena.slot_of.cpu()
                for e in range(cfg.n_routed + cfg.n_shared):
                    nm = mo + (f"experts.{e}." if e < cfg.n_routed else f"shared.{e - cfg.n_routed}.")
                    g, u, d = arena.read_expert(int(so[e]), fmt)
                    out[nm + "gate"], out[nm + "up"], out[nm + "down"] = cpu(g), cpu(u), cpu(d)
            else:
                f = p + "mlp."
                w = cpu(L["mlp_gu"].dequant())
                out[f + "gate"], out[f + "up"] = w[: cfg.dense_inter], w[cfg.dense_inter:]
                out[f + "down"] = cpu(L["mlp_down"].dequant())
        return out
