"""Prepacked expert store: every routed / shared expert as one file holding exactly the bytes of its device slot
(gate | up | down weights, scales, per-tensor tail; layout = ``expert_layout``), so loading an expert is a single
read into pinned memory followed by one host->device copy - no parsing, no re-quantisation.

    <dir>/manifest.json                      format version, model shape, quantisation, slot geometry, per-file sizes + digests
    <dir>/L<layer>/expert_<e>.bin            slot image (stride bytes)

Writing is streaming and resumable: a file is written under a temporary name, fsynced and renamed; a re-run skips
files whose size and digest already match the manifest.  ``PrepackedSource`` reads through mmap (default), pread or
O_DIRECT into caller-provided (pinned) buffers.
Reference: ExpertPrepacker / PrepackedSource / Manifest (src/model/weight_pipeline/*, manifest v9.69.0).  The slot
layout differs (it is this engine's), the contract is the same.
"""
from __future__ import annotations

import hashlib
import json
import mmap
import os
from typing import Dict, Iterable, Optional, Tuple

import torch

FORMAT_VERSION = "lsb200-prepack-1"


def _digest(buf: memoryview) -> str:
    return hashlib.blake2b(buf, digest_size=16).hexdigest()


class PrepackWriter:
    def __init__(self, directory: str, cfg, expert_quant: str, verify_existing: bool = True):
        from ..models.device_model import expert_layout
        self.dir, self.cfg, self.quant = directory, cfg, expert_quant
        self.ef = expert_layout(expert_quant, cfg.hidden, cfg.moe_inter)
        self.verify = verify_existing
        os.makedirs(directory, exist_ok=True)
        self.manifest_path = os.path.join(directory, "manifest.json")
        self.files: Dict[str, dict] = {}
        if os.path.exists(self.manifest_path):
            old = json.load(open(self.manifest_path))
            if old.get("version") == FORMAT_VERSION and old.get("quant") == expert_quant and old.get("stride") == self.ef.stride \
                    and old.get("hidden") == cfg.hidden and old.get("moe_inter") == cfg.moe_inter:
                self.files = old.get("files", {})
        self.written = self.skipped = 0

    def path(self, layer: int, expert: int) -> str:
        return os.path.join(self.dir, f"L{layer:03d}", f"expert_{expert:04d}.bin")

    def add(self, layer: int, expert: int, slot_image: torch.Tensor):
        """``slot_image``: uint8 tensor of ``stride`` bytes (CPU or GPU)."""
        img = slot_image.detach().cpu().contiguous().view(torch.uint8)
        assert img.numel() == self.ef.stride, (img.numel(), self.ef.stride)
        key = f"{layer}/{expert}"
        mv = memoryview(img.numpy())
        dg = _digest(mv)
        p = self.path(layer, expert)
        ent = self.files.get(key)
        if ent and ent["digest"] == dg and os.path.exists(p) and os.path.getsize(p) == self.ef.stride:
            self.skipped += 1
            return
        os.makedirs(os.path.dirname(p), exist_ok=True)
        tmp = p + ".tmp"
        with open(tmp, "wb") as fh:
            fh.write(mv)
            fh.flush()
            os.fsync(fh.fileno())
        os.replace(tmp, p)
        self.files[key] = {"digest": dg, "bytes": self.ef.stride}
        self.written += 1
        if self.written % 64 == 0:
            self.flush()                                   # a crash loses at most the last few files' manifest entries

    def flush(self):
        c = self.cfg
        man = {"version": FORMAT_VERSION, "quant": self.quant, "hidden": c.hidden, "moe_inter": c.moe_inter, "stride": int(self.ef.stride),
               "n_routed": c.n_routed, "n_shared": c.n_shared, "n_layers": c.n_layers, "architecture": c.architecture,
               "layout": {k: int(getattr(self.ef, k)) for k in ("off_gate", "off_up", "off_down", "off_sg", "off_su", "off_sd", "off_tail")},
               "files": self.files}
        tmp = self.manifest_path + ".tmp"
        with open(tmp, "w") as fh:
            json.dump(man, fh)
            fh.flush()
            os.fsync(fh.fileno())
        os.replace(tmp, self.manifest_path)

    def close(self):
        self.flush()


class PrepackedSource:
    def __init__(self, directory: str, mode: str = "mmap"):
        assert mode in ("mmap", "pread", "direct")
        self.dir, self.mode = directory, mode
        self.manifest = json.load(open(os.path.join(directory, "manifest.json")))
        if self.manifest.get("version") != FORMAT_VERSION:
            raise ValueError(f"unsupported prepack version {self.manifest.get('version')!r}")
        self.stride = int(self.manifest["stride"])
        self.quant = self.manifest["quant"]

    def has(self, layer: int, expert: int) -> bool:
        return f"{layer}/{expert}" in self.manifest["files"]

    def path(self, layer: int, expert: int) -> str:
        return os.path.join(self.dir, f"L{layer:03d}", f"expert_{expert:04d}.bin")

    def check_shape(self, cfg, expert_quant: str):
        m = self.manifest
        if (m["hidden"], m["moe_inter"], m["quant"]) != (cfg.hidden, cfg.moe_inter, expert_quant):
            raise ValueError(f"prepacked store is for hidden={m['hidden']} inter={m['moe_inter']} quant={m['quant']}")

    def read_into(self, layer: int, expert: int, dst: torch.Tensor, verify: bool = False):
        """Read one slot image into ``dst`` (uint8 CPU tensor of ``stride`` bytes, ideally pinned)."""
        assert dst.numel() == self.stride and dst.dtype == torch.uint8 and dst.device.type == "cpu"
        p = self.path(layer, expert)
        out = memoryview(dst.numpy())
        if self.mode == "mmap":
            with open(p, "rb") as fh, mmap.mmap(fh.fileno(), 0, access=mmap.ACCESS_READ) as mm:
                out[:] = mm[: self.stride]
        else:
            flags = os.O_RDONLY
            aligned = self.mode == "direct" and dst.data_ptr() % 4096 == 0 and self.stride % 4096 == 0
            if aligned:
                flags |= os.O_DIRECT
            try:
                fd = os.open(p, flags)
            except OSError:
                fd = os.open(p, os.O_RDONLY)               # file system without O_DIRECT
            try:
                off = 0
                while off < self.stride:
                    n = os.preadv(fd, [out[off:]], off)
                    if n <= 0:
                        raise IOError(f"short read of {p}")
                    off += n
            finally:
                os.close(fd)
        if verify and _digest(out) != self.manifest["files"][f"{layer}/{expert}"]["digest"]:
            raise IOError(f"digest mismatch in {p}")

    def verify_all(self) -> Tuple[int, int]:
        """(files checked, files bad)."""
        bad = 0
        buf = torch.empty(self.stride, dtype=torch.uint8)
        for key in self.manifest["files"]:
            layer, expert = (int(v) for v in key.split("/"))
            try:
                self.read_into(layer, expert, buf, verify=True)
            except (IOError, OSError):
                bad += 1
        return len(self.manifest["files"]), bad


def prepack_model(cfg, weights, directory: str, expert_quant: Optional[str] = None, device: str = "cpu") -> PrepackWriter:
    """Quantise every expert of ``weights`` (canonical names, mapping-like: a lazy checkpoint works) into ``directory``."""
    from ..models.device_model import ExpertArena, QLinear, expert_layout
    eq = expert_quant or cfg.expert_quant
    wr = PrepackWriter(directory, cfg, eq)
    ar = ExpertArena(expert_layout(eq, cfg.hidden, cfg.moe_inter), 1, 1, device)
    for i in range(cfg.n_layers):
        if not cfg.is_moe_layer(i):
            continue
        for e in range(cfg.n_routed + cfg.n_shared):
            nm = f"layers.{i}.moe." + (f"experts.{e}." if e < cfg.n_routed else f"shared.{e - cfg.n_routed}.")
            ar.data.zero_()
            ar.write_expert(0, *(QLinear.from_float(weights[nm + t], eq, device) for t in ("gate", "up", "down")))
            wr.add(i, e, ar.data[0])
    wr.close()
    return wr


def load_experts(model, source: PrepackedSource):
    """Fill the model's expert arenas from a prepacked store: one read + one host->device copy per owned expert."""
    cfg = model.cfg
    stage = torch.empty(2, source.stride, dtype=torch.uint8).pin_memory() if torch.cuda.is_available() else torch.empty(2, source.stride, dtype=torch.uint8)
    ev = [None, None]
    k = 0
    for i, L in enumerate(model.layers):
        if "arena" not in L:
            continue
        ar = L["arena"]
        assert ar.ef.stride == source.stride
        so = ar.slot_of.cpu().tolist()
        for e, slot in enumerate(so):
            if slot < 0:
                continue
            b = k & 1
            if ev[b] is not None:
                ev[b].synchronize()
            source.read_into(i, e, stage[b])
            ar.data[slot].copy_(stage[b], non_blocking=True)
            if ar.data.is_cuda:
                ev[b] = torch.cuda.Event()
                ev[b].record()
            k += 1
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    return k
