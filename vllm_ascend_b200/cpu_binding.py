"""NUMA-aware CPU pinning of a rank's process.

Each rank is bound to a slice of the cores of the NUMA node its GPU hangs off, leaving the
node's first cores to interrupt handling, so scheduler/runner threads do not migrate across
sockets.  Policy of vllm_ascend/cpu_binding.py:62-809 (topology discovery → allowed cpus →
per-device slices → ``sched_setaffinity``), with the GPU's node taken from its PCI sysfs
entry instead of the vendor tool.  Every source of topology is injectable so the logic is
tested without hardware.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Callable, Optional

from .logger import logger


def parse_cpu_list(text: str) -> list[int]:
    """"0-3,8,10-11" -> [0,1,2,3,8,10,11]"""
    out: list[int] = []
    for part in text.strip().split(","):
        part = part.strip()
        if not part:
            continue
        if "-" in part:
            a, b = part.split("-")
            out.extend(range(int(a), int(b) + 1))
        else:
            out.append(int(part))
    return sorted(set(out))


def format_cpu_list(cpus: list[int]) -> str:
    cpus = sorted(cpus)
    runs, i = [], 0
    while i < len(cpus):
        j = i
        while j + 1 < len(cpus) and cpus[j + 1] == cpus[j] + 1:
            j += 1
        runs.append(f"{cpus[i]}-{cpus[j]}" if j > i else f"{cpus[i]}")
        i = j + 1
    return ",".join(runs)


@dataclass
class Topology:
    node_cpus: dict[int, list[int]]       # NUMA node -> cpus
    gpu_node: dict[int, int]              # GPU index -> NUMA node (-1 unknown)
    allowed: list[int]                    # cpus this process may use (cgroup / taskset)


def _read(path: str) -> Optional[str]:
    try:
        with open(path) as f:
            return f.read()
    except OSError:
        return None


def discover(num_gpus: int, read: Callable[[str], Optional[str]] = _read,
             pci_bus_ids: Optional[list[str]] = None) -> Topology:
    nodes: dict[int, list[int]] = {}
    online = read("/sys/devices/system/node/online")
    for n in (parse_cpu_list(online) if online else []):
        txt = read(f"/sys/devices/system/node/node{n}/cpulist")
        if txt:
            nodes[n] = parse_cpu_list(txt)
    if not nodes:
        nodes[0] = sorted(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else list(range(os.cpu_count() or 1))
    if pci_bus_ids is None:
        pci_bus_ids = _gpu_bus_ids(num_gpus)
    gpu_node = {}
    for i in range(num_gpus):
        node = -1
        if i < len(pci_bus_ids) and pci_bus_ids[i]:
            bus = pci_bus_ids[i].lower()
            if bus.count(":") == 2 and len(bus.split(":")[0]) == 8:      # NVML pads the domain to 8 hex digits
                bus = bus[4:]
            txt = read(f"/sys/bus/pci/devices/{bus}/numa_node")
            if txt is not None:
                try:
                    node = int(txt.strip())
                except ValueError:
                    node = -1
        gpu_node[i] = node
    allowed = sorted(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else sorted(
        c for cs in nodes.values() for c in cs)
    return Topology(nodes, gpu_node, allowed)


def _gpu_bus_ids(num_gpus: int) -> list[str]:
    try:
        import pynvml
        pynvml.nvmlInit()
        try:
            out = []
            for i in range(num_gpus):
                info = pynvml.nvmlDeviceGetPciInfo(pynvml.nvmlDeviceGetHandleByIndex(i))
                b = info.busId
                out.append(b.decode() if isinstance(b, bytes) else b)
            return out
        finally:
            pynvml.nvmlShutdown()
    except Exception:
        return []


def plan(topo: Topology, local_world: int, reserve_per_node: int = 2) -> dict[int, list[int]]:
    """GPU index -> cpus.  GPUs of one NUMA node split that node's allowed cpus evenly (after
    ``reserve_per_node`` cpus kept free for interrupts); a GPU whose node is unknown, or whose
    node has no allowed cpu, takes an even slice of everything allowed."""
    allowed = set(topo.allowed)
    by_node: dict[int, list[int]] = {}
    for g in range(local_world):
        by_node.setdefault(topo.gpu_node.get(g, -1), []).append(g)
    out: dict[int, list[int]] = {}
    leftovers: list[int] = []
    for node, gpus in by_node.items():
        cpus = [c for c in topo.node_cpus.get(node, []) if c in allowed]
        if node < 0 or not cpus:
            leftovers.extend(gpus)
            continue
        if len(cpus) > reserve_per_node + len(gpus):
            cpus = cpus[reserve_per_node:]
        per = max(1, len(cpus) // len(gpus))
        for k, g in enumerate(gpus):
            out[g] = cpus[k * per:(k + 1) * per] or cpus
    if leftovers:
        cpus = sorted(allowed)
        per = max(1, len(cpus) // local_world)
        for g in leftovers:
            out[g] = cpus[g * per:(g + 1) * per] or cpus
    return out


def bind_cpus(gpu_index: int, local_world: int = 1, topo: Optional[Topology] = None,
              setaffinity: Optional[Callable] = None) -> list[int]:
    topo = topo or discover(max(local_world, gpu_index + 1))
    cpus = plan(topo, max(local_world, gpu_index + 1)).get(gpu_index) or topo.allowed
    (setaffinity or os.sched_setaffinity)(0, set(cpus))
    logger.info("rank on GPU %d bound to cpus %s (NUMA node %s)", gpu_index, format_cpu_list(cpus),
                topo.gpu_node.get(gpu_index, -1))
    return cpus
