"""HuggingFace safetensors container: memory-mapped reader and a writer (8-byte little-endian
header length, JSON header, raw tensor bytes).  Covers the dtypes the supported checkpoints use,
including the NVFP4 tensor quartet (U8 ``weight`` + F8_E4M3 ``weight_scale`` per 16 columns + F32
``weight_scale_2`` + F32 ``input_scale``) and FP8 block-scaled weights (F8_E4M3 ``weight`` + F32
``weight_scale_inv`` per 128x128 block).
Reference: SafetensorsReader (src/model/weight_loader, mmap/pread) and the handlers for nvfp4 /
fp8 / native checkpoints.
"""
from __future__ import annotations

import json
import mmap
import struct
from typing import Dict, Iterable, Optional, Tuple

import numpy as np
import torch

_DT = {"F32": (torch.float32, 4), "F16": (torch.float16, 2), "BF16": (torch.bfloat16, 2), "I32": (torch.int32, 4),
       "I64": (torch.int64, 8), "U8": (torch.uint8, 1), "I8": (torch.int8, 1), "F8_E4M3": (torch.float8_e4m3fn, 1),
       "F8_E5M2": (torch.float8_e5m2, 1), "BOOL": (torch.bool, 1), "F64": (torch.float64, 8), "I16": (torch.int16, 2)}
_DT_REV = {v[0]: k for k, v in _DT.items()}


class SafetensorsReader:
    def __init__(self, path: str):
        self.path = path
        self.f = open(path, "rb")
        (hlen,) = struct.unpack("<Q", self.f.read(8))
        if hlen > 100 << 20:
            raise ValueError("safetensors header too large")
        self.header = json.loads(self.f.read(hlen))
        self.metadata = self.header.pop("__metadata__", {})
        self.base = 8 + hlen
        self.mm = mmap.mmap(self.f.fileno(), 0, access=mmap.ACCESS_READ)

    def keys(self) -> Iterable[str]:
        return self.header.keys()

    def header_items(self) -> dict:
        """{tensor name: (safetensors dtype string, shape)} of this file."""
        return {k: (e["dtype"], tuple(e["shape"])) for k, e in self.header.items()}

    def info(self, name: str) -> Tuple[str, Tuple[int, ...], int]:
        e = self.header[name]
        return e["dtype"], tuple(e["shape"]), e["data_offsets"][1] - e["data_offsets"][0]

    def get(self, name: str) -> torch.Tensor:
        e = self.header[name]
        dt, sz = _DT[e["dtype"]]
        a, b = e["data_offsets"]
        n = int(np.prod(e["shape"])) if e["shape"] else 1
        if b - a != n * sz:
            raise ValueError(f"{name}: byte range does not match shape")
        buf = np.frombuffer(self.mm, dtype=np.uint8, count=b - a, offset=self.base + a)
        t = torch.from_numpy(buf.copy()).view(dt)
        return t.reshape(e["shape"])

    def close(self):
        self.mm.close()
        self.f.close()


def write_safetensors(path: str, tensors: Dict[str, torch.Tensor], metadata: Optional[Dict[str, str]] = None):
    header, off, blobs = {}, 0, []
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous()
        raw = t.view(torch.uint8).reshape(-1).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _DT_REV[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        off += len(raw)
        blobs.append(raw)
    if metadata:
        header["__metadata__"] = metadata
    h = json.dumps(header, separators=(",", ":")).encode()
    h += b" " * ((8 - len(h) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(h)))
        f.write(h)
        for b in blobs:
            f.write(b)
