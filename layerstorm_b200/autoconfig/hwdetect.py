"""Hardware descriptor for the autoconfig solver and the server boot path.

Reads, never writes: GPU list (name, memory, compute capability, NUMA node, peer reachability)
through NVML when it is importable and a driver is present, else through ``torch.cuda``; host RAM,
core count and NUMA nodes from ``/proc`` and ``/sys``; free space on the configured NVMe paths.
Nothing here changes a GPU setting.  Tests pass a hand-written descriptor instead of probing.
Reference: python/autoconfig/hwdetect.py (same role: the probe that feeds the solver; the
descriptor on B200 is eight identical GPUs on one NVSwitch domain rather than a PCIe tree).
"""
from __future__ import annotations

import hashlib
import json
import os
import shutil
from dataclasses import asdict, dataclass, field


@dataclass
class GpuInfo:
    id: int
    type: str = "b200"
    vram_gb: float = 180.0
    sm_count: int = 148
    cc: str = "10.0"
    numa_node: int = 0
    nvlink: bool = True
    free_gb: float | None = None


@dataclass
class HardwareInfo:
    gpus: list[GpuInfo] = field(default_factory=list)
    system_ram_gb: float = 0.0
    free_ram_gb: float = 0.0
    cpu_cores: int = 0
    numa_nodes: int = 1
    nvme: dict[str, float] = field(default_factory=dict)     # path -> free GB
    p2p_all: bool = True                                     # every GPU pair peer-accessible
    hbm_gbs: float = 6455.0                                  # measured copy bandwidth of one GPU
    nvlink_gbs: float = 770.0                                # measured peer copy, per direction
    h2d_gbs: float = 55.0                                    # pinned host -> device

    def fingerprint(self) -> str:
        """Stable id of the machine shape; a stored autoconfig result is reused only while it matches."""
        key = {"gpus": [(g.type, round(g.vram_gb), g.cc) for g in self.gpus], "ram": round(self.system_ram_gb / 8),
               "numa": self.numa_nodes, "p2p": self.p2p_all}
        return hashlib.sha256(json.dumps(key, sort_keys=True).encode()).hexdigest()[:16]

    def to_dict(self) -> dict:
        return asdict(self)

    @classmethod
    def from_dict(cls, d: dict) -> "HardwareInfo":
        d = dict(d)
        d["gpus"] = [GpuInfo(**g) for g in d.get("gpus", [])]
        return cls(**d)

    def hardware_section(self, roles: dict[int, list[str]] | None = None) -> dict:
        """The ``hardware`` config section for this machine."""
        return {"gpus": [{"id": g.id, "type": g.type, "vram_gb": g.vram_gb, "numa_node": g.numa_node,
                          "roles": (roles or {}).get(g.id, ["attention", "resident", "expert_streaming"])} for g in self.gpus],
                "system_ram_gb": int(self.system_ram_gb), "nvme_paths": sorted(self.nvme)}


def _meminfo() -> tuple[float, float]:
    tot = free = 0.0
    try:
        for line in open("/proc/meminfo"):
            if line.startswith("MemTotal:"):
                tot = float(line.split()[1]) / 1048576
            elif line.startswith("MemAvailable:"):
                free = float(line.split()[1]) / 1048576
    except OSError:
        pass
    return tot, free


def _numa_nodes() -> int:
    try:
        return max(1, sum(1 for d in os.listdir("/sys/devices/system/node") if d.startswith("node") and d[4:].isdigit()))
    except OSError:
        return 1


def _short_name(name: str) -> str:
    n = name.lower()
    for k in ("b200", "b100", "h200", "h100", "gb200", "5090", "5080"):
        if k in n:
            return ("rtx" + k) if k[0] == "5" else k
    return n.replace("nvidia", "").strip().replace(" ", "_") or "gpu"


def _gpus_nvml() -> list[GpuInfo] | None:
    try:
        import pynvml
        pynvml.nvmlInit()
    except Exception:
        return None
    out = []
    try:
        for i in range(pynvml.nvmlDeviceGetCount()):
            h = pynvml.nvmlDeviceGetHandleByIndex(i)
            name = pynvml.nvmlDeviceGetName(h)
            name = name.decode() if isinstance(name, bytes) else name
            mem = pynvml.nvmlDeviceGetMemoryInfo(h)
            try:
                maj, mnr = pynvml.nvmlDeviceGetCudaComputeCapability(h)
            except Exception:
                maj, mnr = 0, 0
            numa = 0
            try:
                bus = pynvml.nvmlDeviceGetPciInfo(h).busId
                bus = bus.decode() if isinstance(bus, bytes) else bus
                p = f"/sys/bus/pci/devices/{bus.lower()[-12:]}/numa_node"
                if os.path.exists(p):
                    numa = max(0, int(open(p).read().strip()))
            except Exception:
                pass
            nvl = False
            try:
                nvl = pynvml.nvmlDeviceGetNvLinkState(h, 0) == 1
            except Exception:
                pass
            out.append(GpuInfo(id=i, type=_short_name(name), vram_gb=mem.total / 2**30, free_gb=mem.free / 2**30,
                               cc=f"{maj}.{mnr}", numa_node=numa, nvlink=nvl, sm_count=0))
    finally:
        try:
            pynvml.nvmlShutdown()
        except Exception:
            pass
    return out


def _gpus_torch() -> list[GpuInfo]:
    try:
        import torch
        if not torch.cuda.is_available():
            return []
        out = []
        for i in range(torch.cuda.device_count()):
            p = torch.cuda.get_device_properties(i)
            out.append(GpuInfo(id=i, type=_short_name(p.name), vram_gb=p.total_memory / 2**30, sm_count=p.multi_processor_count,
                               cc=f"{p.major}.{p.minor}"))
        return out
    except Exception:
        return []


def detect(nvme_paths: list[str] | None = None) -> HardwareInfo:
    gpus = _gpus_nvml()
    if not gpus:
        gpus = _gpus_torch()
    tot, free = _meminfo()
    nv = {}
    for p in nvme_paths or []:
        try:
            nv[p] = shutil.disk_usage(p).free / 1e9
        except OSError:
            pass
    return HardwareInfo(gpus=gpus, system_ram_gb=tot, free_ram_gb=free, cpu_cores=os.cpu_count() or 0,
                        numa_nodes=_numa_nodes(), nvme=nv, p2p_all=all(g.nvlink for g in gpus) if gpus else False)


def synthetic(n_gpus: int = 8, vram_gb: float = 180.0, ram_gb: float = 2048.0, gpu_type: str = "b200") -> HardwareInfo:
    """A descriptor for tests and for `--autoconfig` dry runs on a machine without GPUs."""
    return HardwareInfo(gpus=[GpuInfo(id=i, type=gpu_type, vram_gb=vram_gb, numa_node=i * 2 // max(n_gpus, 1)) for i in range(n_gpus)],
                        system_ram_gb=ram_gb, free_ram_gb=ram_gb * 0.95, cpu_cores=128, numa_nodes=2)
