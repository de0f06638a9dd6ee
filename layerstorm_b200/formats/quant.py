"""Weight quantisation codecs (torch, device-agnostic): FP8 e4m3 with 128x128 block scales
and NVFP4 (E2M1 values, e4m3 scale per 16 columns in the 128x4 scale-atom layout, fp32
per-tensor scale).  Each codec has a quantiser and an exact dequantiser; the dequantiser is
the oracle for the CUDA kernels that consume these layouts.

Reference formats: FP8 blockwise scale grid tests/unit/fp8_gemm_test.cpp:129-153; NVFP4
slot layout deps/LayerStoRmCpuExpertKernels/csrc/compute/cpu/nvfp4_cpu_kernel.h:14-30 and the
scale-atom index src/model/weight_loader/nvfp4_sfb_reformat.h:10-18.
"""
from __future__ import annotations

import torch

FP4_VALUES = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])
_FP4_MID = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0])


# ---------------------------------------------------------------- FP8 block-128
def quantize_fp8_block(w: torch.Tensor, block: int = 128, pow2: bool = True):
    """w [N,K] float -> (uint8 e4m3 [N,K], fp32 scales [ceil(N/b), ceil(K/b)]).  ``pow2``: scales rounded up to powers of two
    (the UE8M0 scale convention of DeepSeek-V3.1+ FP8 checkpoints; lets the block-scaled tensor-core path take the weights as
    they are - E4M3 is a floating-point format, so the rounding costs range, not relative precision)."""
    N, K = w.shape
    nb, kb = (N + block - 1) // block, (K + block - 1) // block
    wp = torch.zeros(nb * block, kb * block, dtype=torch.float32, device=w.device)
    wp[:N, :K] = w.float()
    blocks = wp.view(nb, block, kb, block)
    amax = blocks.abs().amax(dim=(1, 3)).clamp_min(1e-12)
    scale = amax / 448.0
    if pow2:
        scale = torch.exp2(torch.ceil(torch.log2(scale)))
    q = (blocks / scale[:, None, :, None]).view(nb * block, kb * block)[:N, :K]
    q8 = q.contiguous().to(torch.float8_e4m3fn).view(torch.uint8)
    return q8, scale.contiguous()


def dequantize_fp8_block(q8: torch.Tensor, scale: torch.Tensor, block: int = 128) -> torch.Tensor:
    N, K = q8.shape
    w = q8.view(torch.float8_e4m3fn).float()
    s = scale.repeat_interleave(block, 0)[:N].repeat_interleave(block, 1)[:, :K]
    return w * s


# ---------------------------------------------------------------- NVFP4
def sf_atom_size(N: int, K: int) -> int:
    G = K // 16
    return ((N + 127) // 128) * ((G + 3) // 4) * 512


def sf_atom_index(n: torch.Tensor, g: torch.Tensor, K: int) -> torch.Tensor:
    gt = ((K // 16) + 3) // 4
    return ((n // 128) * gt + g // 4) * 512 + (n % 32) * 16 + ((n % 128) // 32) * 4 + g % 4


def e4m3_round(x: torch.Tensor) -> torch.Tensor:
    return x.to(torch.float8_e4m3fn).float()


def quantize_nvfp4(w: torch.Tensor):
    """w [N,K] (K % 32 == 0) -> (packed uint8 [N,K/2], scale atoms uint8 [sf_atom_size], fp32 global scale)."""
    N, K = w.shape
    assert K % 32 == 0
    dev = w.device
    wf = w.float()
    G = K // 16
    gs = float(wf.abs().max().clamp_min(1e-12)) / (448.0 * 6.0)
    blocks = wf.view(N, G, 16)
    sf = e4m3_round((blocks.abs().amax(-1) / (6.0 * gs)).clamp(max=448.0))
    sf = torch.where(sf == 0, torch.full_like(sf, 2.0 ** -9), sf)
    v = blocks / (sf[..., None] * gs)
    mag = torch.bucketize(v.abs(), _FP4_MID.to(dev))          # 0..7
    code = (mag | ((v < 0).to(torch.int64) << 3)).view(N, K).to(torch.uint8)
    packed = (code[:, 0::2] | (code[:, 1::2] << 4)).contiguous()
    atoms = torch.zeros(sf_atom_size(N, K), dtype=torch.uint8, device=dev)
    n_idx = torch.arange(N, device=dev)[:, None].expand(N, G)
    g_idx = torch.arange(G, device=dev)[None, :].expand(N, G)
    atoms[sf_atom_index(n_idx, g_idx, K).reshape(-1)] = sf.to(torch.float8_e4m3fn).view(torch.uint8).reshape(-1)
    return packed, atoms, gs


def dequantize_nvfp4(packed: torch.Tensor, atoms: torch.Tensor, gs: float, N: int, K: int) -> torch.Tensor:
    dev = packed.device
    lo = (packed & 0xF).to(torch.int64)
    hi = (packed >> 4).to(torch.int64)
    code = torch.stack((lo, hi), -1).view(N, K)
    val = FP4_VALUES.to(dev)[code & 7] * torch.where((code & 8) != 0, -1.0, 1.0)
    G = K // 16
    n_idx = torch.arange(N, device=dev)[:, None].expand(N, G)
    g_idx = torch.arange(G, device=dev)[None, :].expand(N, G)
    sf = atoms[sf_atom_index(n_idx, g_idx, K)].view(torch.float8_e4m3fn).float()
    return (val.view(N, G, 16) * sf[..., None] * gs).view(N, K)


def random_nvfp4_(packed: torch.Tensor, atoms: torch.Tensor, gen=None):
    """Fill pre-allocated NVFP4 storage with random nibbles and benign scales (0.5..0.94) in place;
    with a global scale of ~0.0095 the dequantised weights have a standard deviation near 0.02."""
    packed.random_(0, 256, generator=gen)
    atoms.random_(0x30, 0x40, generator=gen)
    return 0.02 / 2.1
