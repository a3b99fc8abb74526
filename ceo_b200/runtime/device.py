"""Device, stream/event and topology layer: what the reference keeps in src/runtime/cuda.zig
(`DeviceProp` 198-278, `CudaStream` 291-314, `CudaEvent` 317-351, `CudaDevice.isBlackwell`
354-402, `CudaInit` 405-454) and src/runtime/main.zig (`DistributedRuntime` 141-319,
`Topology.detect` 322-391 - there a fake with one NUMA node and PCI bus = index).

PyTorch owns the CUDA context, so these are thin, typed views over ``torch.cuda``; the topology
is read for real from NVML (PCI ids, NVLink state) and sysfs (NUMA nodes, CPU lists), each
source optional and injectable so the logic is testable without a GPU.  Nothing here changes
a device setting: every NVML call is a query.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from pathlib import Path

import torch

from ..utils.errors import (InvalidWorldSize, NoGpuAvailable, PeerAccessUnavailable,
                            UnsupportedDevice)


@dataclass
class DeviceInfo:
    index: int
    name: str
    major: int
    minor: int
    sm_count: int
    total_memory: int
    l2_bytes: int = 0
    smem_per_block_optin: int = 0

    @property
    def is_blackwell(self) -> bool:
        """Compute capability 10.x or later (the reference's test: major >= 10)."""
        return self.major >= 10

    @property
    def is_sm100(self) -> bool:
        """Exactly the architecture the kernel library is compiled for (sm_100a)."""
        return self.major == 10 and self.minor == 0


def device_count() -> int:
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def device_info(index: int = 0) -> DeviceInfo:
    if index >= device_count():
        raise NoGpuAvailable(f"no CUDA device {index}")
    p = torch.cuda.get_device_properties(index)
    return DeviceInfo(index, p.name, p.major, p.minor, p.multi_processor_count, p.total_memory,
                      getattr(p, "L2_cache_size", 0),
                      getattr(p, "shared_memory_per_block_optin", 0))


def memory_info(index: int = 0) -> tuple[int, int]:
    """(free, total) bytes on the device."""
    return torch.cuda.mem_get_info(index)


def require_sm100(index: int = 0) -> DeviceInfo:
    """The kernel library holds sm_100a code only; fail early and clearly anywhere else."""
    info = device_info(index)
    if not info.is_sm100:
        raise UnsupportedDevice(f"{info.name} is sm_{info.major}{info.minor}; the kernels are built "
                            "for sm_100a (B200) only")
    return info


class Stream:
    """A non-blocking stream on one device (CudaStream of the reference)."""

    def __init__(self, device: int = 0, priority: int = 0):
        self.device = device
        self.stream = torch.cuda.Stream(device=device, priority=priority)

    @property
    def handle(self) -> int:
        return self.stream.cuda_stream

    def synchronize(self):
        self.stream.synchronize()

    def wait_event(self, ev: "Event"):
        self.stream.wait_event(ev.event)

    def __enter__(self):
        self._ctx = torch.cuda.stream(self.stream)
        self._ctx.__enter__()
        return self

    def __exit__(self, *exc):
        return self._ctx.__exit__(*exc)


class Event:
    """A timing event (CudaEvent of the reference)."""

    def __init__(self, timing: bool = True):
        self.event = torch.cuda.Event(enable_timing=timing)

    def record(self, stream: Stream | None = None):
        self.event.record(stream.stream if stream is not None else None)

    def synchronize(self):
        self.event.synchronize()

    def elapsed_ms(self, end: "Event") -> float:
        return self.event.elapsed_time(end.event)


# ---- topology -------------------------------------------------------------------------------

@dataclass
class NumaNode:
    id: int
    cpus: list[int] = field(default_factory=list)
    gpus: list[int] = field(default_factory=list)
    memory_size: int = 0


@dataclass
class GpuAffinity:
    gpu_id: int
    numa_node: int
    pci_domain: int = 0
    pci_bus: int = 0
    pci_device: int = 0
    nvlink_active: int = 0          # active NVLink links (0 when unknown)


def parse_cpulist(text: str) -> list[int]:
    """'0-3,8,10-11' -> [0,1,2,3,8,10,11]"""
    out: list[int] = []
    for part in text.strip().split(","):
        if not part:
            continue
        if "-" in part:
            a, b = part.split("-")
            out.extend(range(int(a), int(b) + 1))
        else:
            out.append(int(part))
    return out


class _Nvml:
    """The handful of NVML queries the topology needs; absent library = no information."""

    def __init__(self):
        import pynvml
        self.n = pynvml
        pynvml.nvmlInit()

    def count(self) -> int:
        return self.n.nvmlDeviceGetCount()

    def pci(self, i: int) -> tuple[int, int, int, str]:
        h = self.n.nvmlDeviceGetHandleByIndex(i)
        p = self.n.nvmlDeviceGetPciInfo(h)
        bus_id = p.busId.decode() if isinstance(p.busId, bytes) else p.busId
        return p.domain, p.bus, p.device, bus_id

    def nvlinks(self, i: int) -> int:
        h = self.n.nvmlDeviceGetHandleByIndex(i)
        active = 0
        for link in range(18):
            try:
                if self.n.nvmlDeviceGetNvLinkState(h, link):
                    active += 1
            except Exception:
                break
        return active


class Topology:
    """NUMA nodes and per-GPU affinity of this host."""

    def __init__(self, numa_nodes: list[NumaNode], gpu_affinity: list[GpuAffinity]):
        self.numa_nodes, self.gpu_affinity = numa_nodes, gpu_affinity

    @classmethod
    def detect(cls, num_gpus: int | None = None, nvml=None, sysfs: str = "/sys") -> "Topology":
        """``nvml``: an object with count()/pci(i)/nvlinks(i) (default: the NVML library when
        it loads); ``sysfs``: root of a sysfs tree.  With neither source every GPU lands on
        NUMA node 0 with PCI bus = index, which is all the reference ever reports."""
        if nvml is None:
            try:
                nvml = _Nvml()
            except Exception:
                nvml = None
        if num_gpus is None:
            num_gpus = nvml.count() if nvml is not None else device_count()
        root = Path(sysfs)
        nodes: dict[int, NumaNode] = {}
        node_dir = root / "devices" / "system" / "node"
        if node_dir.is_dir():
            for d in sorted(node_dir.glob("node[0-9]*")):
                nid = int(d.name[4:])
                cpus, mem = [], 0
                try:
                    cpus = parse_cpulist((d / "cpulist").read_text())
                except OSError:
                    pass
                try:
                    for line in (d / "meminfo").read_text().splitlines():
                        if "MemTotal" in line:
                            mem = int(line.split()[-2]) * 1024
                except (OSError, ValueError, IndexError):
                    pass
                nodes[nid] = NumaNode(nid, cpus, [], mem)
        if not nodes:
            nodes[0] = NumaNode(0, list(range(os.cpu_count() or 1)), [], 0)
        aff = []
        for i in range(num_gpus):
            dom, bus, dev, links, numa = 0, i, 0, 0, 0
            if nvml is not None:
                try:
                    dom, bus, dev, bus_id = nvml.pci(i)
                    links = nvml.nvlinks(i)
                    # sysfs names devices with a 4-digit domain; NVML prints 8 digits
                    short = bus_id.lower()[-12:]
                    f = root / "bus" / "pci" / "devices" / short / "numa_node"
                    if f.exists():
                        numa = max(int(f.read_text().strip()), 0)
                except Exception:
                    pass
            if numa not in nodes:
                numa = min(nodes)
            nodes[numa].gpus.append(i)
            aff.append(GpuAffinity(i, numa, dom, bus, dev, links))
        return cls([nodes[k] for k in sorted(nodes)], aff)

    def gpu_for_numa(self, numa_node: int) -> int | None:
        for a in self.gpu_affinity:
            if a.numa_node == numa_node:
                return a.gpu_id
        return None

    def cpus_for_gpu(self, gpu: int) -> list[int]:
        node = self.gpu_affinity[gpu].numa_node
        for n in self.numa_nodes:
            if n.id == node:
                return n.cpus
        return []


def peer_access_matrix(n: int | None = None) -> list[list[bool]]:
    """m[i][j]: device i can map device j's memory (what the IPC buffers of the fused
    collectives need; the reference's enablePeerAccess loops over the same pairs,
    src/runtime/main.zig:310-318)."""
    n = device_count() if n is None else n
    return [[i == j or torch.cuda.can_device_access_peer(i, j) for j in range(n)]
            for i in range(n)]


class DistributedRuntime:
    """One process per GPU: binds the device, joins the process group, and answers the
    reference's runtime queries (src/runtime/main.zig:141-319)."""

    def __init__(self, rank: int, world_size: int, local_rank: int, comm=None):
        self.rank, self.world_size, self.local_rank, self.comm = rank, world_size, local_rank, comm
        self.device = device_info(local_rank) if device_count() else None
        self.stream = Stream(local_rank) if device_count() else None

    @classmethod
    def init_single_gpu(cls) -> "DistributedRuntime":
        if device_count() == 0:
            raise NoGpuAvailable("no CUDA device")
        torch.cuda.set_device(0)
        return cls(0, 1, 0)

    @classmethod
    def init(cls, runtime_cfg=None) -> "DistributedRuntime":
        """Joins the job the launcher described (RANK / WORLD_SIZE / LOCAL_RANK); the configured
        ``world_size`` must match it."""
        from ..parallel.comm import Comm, init_distributed
        rank, world, local = init_distributed()
        want = getattr(runtime_cfg, "world_size", None)
        if want is not None and want == 0:
            raise InvalidWorldSize("runtime.world_size is 0")
        if want not in (None, world) and world > 1:
            raise InvalidWorldSize(f"launched with {world} ranks, config says {want}")
        if device_count():
            torch.cuda.set_device(local)
        return cls(rank, world, local, Comm() if world > 1 else None)

    def synchronize(self):
        if device_count():
            torch.cuda.synchronize()
        if self.comm is not None:
            self.comm.barrier()

    def get_memory_info(self) -> tuple[int, int]:
        return memory_info(self.local_rank)

    def all_blackwell(self) -> bool:
        ok = self.device is not None and self.device.is_blackwell
        if self.comm is None:
            return ok
        t = torch.tensor([1.0 if ok else 0.0],
                         device="cuda" if device_count() else "cpu")
        import torch.distributed as dist
        self.comm.all_reduce(t, op=dist.ReduceOp.MIN)
        return bool(t.item() > 0.5)

    def enable_peer_access(self) -> list[list[bool]]:
        """Peer mappings are made when symmetric buffers are opened; this checks up front
        that every pair of this node's devices allows it."""
        m = peer_access_matrix()
        bad = [(i, j) for i, r in enumerate(m) for j, ok in enumerate(r) if not ok]
        if bad:
            raise PeerAccessUnavailable(f"no peer access between {bad[:4]}")
        return m
