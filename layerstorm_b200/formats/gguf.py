"""GGUF v3 files: reading (memory-mapped, native parser), writing, and the ggml block codecs.

The container parser and the k-quant / MXFP4 codecs are C++ (csrc/runtime/gguf.cpp); this module
wraps them with NumPy views.  Reference: GgufReader (src/model/weight_loader/gguf_reader.cpp) and
the block specs of src/model/quantization/gguf_kquant.h:49-57.
"""
from __future__ import annotations

import ctypes
from typing import Dict, List, Optional, Tuple

import numpy as np

from ..runtime import native as nt

GGML_TYPES = {"F32": 0, "F16": 1, "Q8_0": 8, "Q2_K": 10, "Q3_K": 11, "Q4_K": 12, "Q5_K": 13, "Q6_K": 14, "I32": 26, "BF16": 30, "MXFP4": 39}
GGML_NAMES = {v: k for k, v in GGML_TYPES.items()}


def block_elems(t: int) -> int:
    return nt.load().lsb_ggml_block_elems(t)


def block_bytes(t: int) -> int:
    return nt.load().lsb_ggml_block_bytes(t)


def nbytes_for(t: int, n_elements: int) -> int:
    be = block_elems(t)
    if be == 0 or n_elements % be:
        raise ValueError(f"type {t} cannot hold {n_elements} elements")
    return n_elements // be * block_bytes(t)


def dequantize(t: int, raw: np.ndarray, n_elements: int) -> np.ndarray:
    raw = np.ascontiguousarray(raw.view(np.uint8))
    out = np.empty(n_elements, dtype=np.float32)
    rc = nt.load().lsb_ggml_dequantize(t, raw.ctypes.data, out.ctypes.data, n_elements)
    if rc:
        raise nt.NativeError(rc, f"dequantize type {t}")
    return out


def quantize(t: int, x: np.ndarray) -> np.ndarray:
    if t == GGML_TYPES["I32"]:
        return np.ascontiguousarray(np.asarray(x).astype(np.int32).reshape(-1)).view(np.uint8)
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1)
    out = np.empty(nbytes_for(t, x.size), dtype=np.uint8)
    rc = nt.load().lsb_ggml_quantize(t, x.ctypes.data, out.ctypes.data, x.size)
    if rc:
        raise nt.NativeError(rc, f"quantize type {t}")
    return out


# ---- block types the GPU kernels read without re-quantisation, and their device layouts ------------------------------
# Q4_K and Q5_K blocks are multiples of 16 bytes and are used as they sit in the file.  Q6_K blocks (210 bytes) are padded
# to 224 so that every field is 16-byte aligned; Q8_0 rows are split into a plane of quants and a plane of fp16 scales (the
# file puts a 2-byte scale in front of every 32 quants).  Both re-layouts move bytes only: values are bit-identical.
DEVICE_NATIVE = {12: "gguf_q4_k", 13: "gguf_q5_k", 14: "gguf_q6_k", 8: "gguf_q8_0"}
DEVICE_TYPE_OF = {v: k for k, v in DEVICE_NATIVE.items()}
Q6K_DEVICE_BLOCK = 224


def device_row_bytes(t: int, K: int) -> int:
    if t == 12:
        return K // 256 * 144
    if t == 13:
        return K // 256 * 176
    if t == 14:
        return K // 256 * Q6K_DEVICE_BLOCK
    if t == 8:
        return K + K // 16
    raise ValueError(f"ggml type {t} has no device layout")


def to_device_layout(t: int, raw: np.ndarray, N: int, K: int) -> np.ndarray:
    """File-order blocks of an [N, K] tensor -> uint8 [N, device_row_bytes]."""
    raw = np.ascontiguousarray(raw).view(np.uint8).reshape(-1)
    if K % 256:
        raise ValueError("device layouts need K % 256 == 0")
    if t in (12, 13):
        return raw.reshape(N, -1)
    if t == 14:
        nb = N * K // 256
        out = np.zeros((nb, Q6K_DEVICE_BLOCK), dtype=np.uint8)
        out[:, :210] = raw.reshape(nb, 210)
        return out.reshape(N, -1)
    if t == 8:
        b = raw.reshape(N, K // 32, 34)
        return np.ascontiguousarray(np.concatenate([b[:, :, 2:].reshape(N, K), b[:, :, :2].reshape(N, K // 16)], axis=1))
    raise ValueError(f"ggml type {t} has no device layout")


def from_device_layout(t: int, dev: np.ndarray, N: int, K: int) -> np.ndarray:
    """Inverse of :func:`to_device_layout`: flat file-order blocks."""
    dev = np.ascontiguousarray(dev).view(np.uint8).reshape(N, -1)
    if t in (12, 13):
        return dev.reshape(-1)
    if t == 14:
        return np.ascontiguousarray(dev.reshape(-1, Q6K_DEVICE_BLOCK)[:, :210]).reshape(-1)
    if t == 8:
        q = dev[:, :K].reshape(N, K // 32, 32)
        d = dev[:, K:].reshape(N, K // 32, 2)
        return np.ascontiguousarray(np.concatenate([d, q], axis=2)).reshape(-1)
    raise ValueError(f"ggml type {t} has no device layout")


class GgufReader:
    def __init__(self, path: str):
        self.lib = nt.load()
        rc = ctypes.c_int(0)
        self.h = self.lib.lsb_gguf_open(path.encode(), ctypes.cast(ctypes.pointer(rc), ctypes.c_void_p))
        if not self.h:
            raise nt.NativeError(rc.value, f"open {path}")
        self.path = path
        self.tensors: Dict[str, dict] = {}
        name = ctypes.create_string_buffer(512)
        ty, nd, nb = ctypes.c_int(0), ctypes.c_int(0), ctypes.c_ulonglong(0)
        dims = (ctypes.c_ulonglong * 4)()
        vp = lambda x: ctypes.cast(ctypes.pointer(x), ctypes.c_void_p)
        for i in range(self.lib.lsb_gguf_n_tensors(self.h)):
            self.lib.lsb_gguf_tensor_info(self.h, i, ctypes.cast(name, ctypes.c_void_p), 512, vp(ty), vp(nd), ctypes.cast(dims, ctypes.c_void_p), vp(nb))
            ne = [int(dims[d]) for d in range(nd.value)]
            # ggml lists the fastest dimension first; numpy shape is the reverse
            self.tensors[name.value.decode()] = {"index": i, "type": ty.value, "ne": ne, "shape": tuple(reversed(ne)), "nbytes": int(nb.value)}

    def close(self):
        if self.h:
            self.lib.lsb_gguf_close(self.h)
            self.h = None

    def __del__(self):
        self.close()

    @property
    def version(self) -> int:
        return self.lib.lsb_gguf_version(self.h)

    def meta_keys(self) -> List[str]:
        buf = ctypes.create_string_buffer(512)
        out = []
        for i in range(self.lib.lsb_gguf_n_meta(self.h)):
            self.lib.lsb_gguf_meta_key(self.h, i, ctypes.cast(buf, ctypes.c_void_p), 512)
            out.append(buf.value.decode())
        return out

    def meta(self, key: str, default=None):
        k = key.encode()
        t = self.lib.lsb_gguf_meta_type(self.h, k)
        if t < 0:
            return default
        if t == 8:
            n = self.lib.lsb_gguf_meta_str(self.h, k, None, 0)
            buf = ctypes.create_string_buffer(n + 1)
            self.lib.lsb_gguf_meta_str(self.h, k, ctypes.cast(buf, ctypes.c_void_p), n + 1)
            return buf.value.decode(errors="replace")
        if t == 9:
            n = self.lib.lsb_gguf_meta_arr_len(self.h, k)
            buf = ctypes.create_string_buffer(4096)
            out = []
            for i in range(n):
                ln = self.lib.lsb_gguf_meta_arr_str(self.h, k, i, ctypes.cast(buf, ctypes.c_void_p), 4096)
                out.append(buf.value.decode(errors="replace") if ln >= 0 else self.lib.lsb_gguf_meta_arr_num(self.h, k, i))
            return out
        v = self.lib.lsb_gguf_meta_num(self.h, k)
        return float(v) if t in (6, 12) else (bool(v) if t == 7 else int(v))

    def raw(self, name: str) -> np.ndarray:
        t = self.tensors[name]
        ptr = self.lib.lsb_gguf_tensor_data(self.h, t["index"])
        return np.ctypeslib.as_array(ctypes.cast(ptr, ctypes.POINTER(ctypes.c_uint8)), shape=(t["nbytes"],))

    def get(self, name: str) -> np.ndarray:
        """Dequantised fp32 tensor in NumPy (row-major) shape."""
        t = self.tensors[name]
        n = int(np.prod(t["shape"])) if t["shape"] else 1
        if t["type"] == GGML_TYPES["I32"]:                     # integer tables (hash-layer token -> expert ids) pass through
            return self.raw(name).view(np.int32).reshape(t["shape"]).copy()
        return dequantize(t["type"], self.raw(name), n).reshape(t["shape"])


    def tensor_names(self) -> List[str]:
        return list(self.tensors)

    def tensor_type(self, name: str) -> int:
        return self.tensors[name]["type"]

    def tensor_shape(self, name: str) -> Tuple[int, ...]:
        return self.tensors[name]["shape"]

    def get_slice(self, name: str, elem0: int, n: int) -> np.ndarray:
        """Dequantise ``n`` consecutive elements starting at ``elem0`` (both multiples of the type's
        block size), e.g. one expert out of a stacked ``[E, rows, cols]`` tensor."""
        t = self.tensors[name]
        be, bb = block_elems(t["type"]), block_bytes(t["type"])
        if elem0 % be or n % be:
            raise ValueError(f"slice [{elem0}, +{n}) is not aligned to {be}-element blocks")
        raw = self.raw(name)[elem0 // be * bb: (elem0 + n) // be * bb]
        return dequantize(t["type"], raw, n)


class GgufWriter:
    def __init__(self):
        self.lib = nt.load()
        self.h = self.lib.lsb_gguf_writer_new()
        self._keep = []

    def meta(self, key: str, value):
        k = key.encode()
        if isinstance(value, (list, tuple)) and value and all(isinstance(v, str) for v in value):
            arr = (ctypes.c_char_p * len(value))(*[v.encode() for v in value])
            self.lib.lsb_gguf_writer_meta_str_array(self.h, k, ctypes.cast(arr, ctypes.c_void_p), len(value))
        elif isinstance(value, (list, tuple)):
            arr = (ctypes.c_int * len(value))(*[int(v) for v in value])
            self.lib.lsb_gguf_writer_meta_i32_array(self.h, k, ctypes.cast(arr, ctypes.c_void_p), len(value))
        elif isinstance(value, str):
            self.lib.lsb_gguf_writer_meta_str(self.h, k, value.encode())
        elif isinstance(value, float):
            self.lib.lsb_gguf_writer_meta_f32(self.h, k, value)
        else:
            self.lib.lsb_gguf_writer_meta_u32(self.h, k, int(value))

    def add(self, name: str, array: np.ndarray, ggml_type: int = 0):
        """Quantise ``array`` (fp32, NumPy shape) to ``ggml_type`` and add it."""
        raw = quantize(ggml_type, array)
        self.add_raw(name, raw, ggml_type, array.shape)

    def add_raw(self, name: str, raw: np.ndarray, ggml_type: int, shape: Tuple[int, ...]):
        raw = np.ascontiguousarray(raw.view(np.uint8))
        self._keep.append(raw)
        ne = list(reversed(shape))
        dims = (ctypes.c_ulonglong * 4)(*(ne + [1] * (4 - len(ne))))
        rc = self.lib.lsb_gguf_writer_add_tensor(self.h, name.encode(), ggml_type, len(ne), ctypes.cast(dims, ctypes.c_void_p), raw.ctypes.data, raw.size)
        if rc:
            raise nt.NativeError(rc, "add_tensor")

    def write(self, path: str):
        rc = self.lib.lsb_gguf_writer_finish(self.h, path.encode())
        self.lib.lsb_gguf_writer_free(self.h)
        self.h = None
        if rc:
            raise nt.NativeError(rc, f"write {path}")
