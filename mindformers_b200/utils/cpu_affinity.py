"""Binding a rank's host threads to the CPU cores next to its GPU.

The reference excludes the cores that the Ascend runtime's work queues occupy and splits the rest between the ranks
of a node (``mindformers/utils/cann_cores_utils.py`` ``get_cann_workqueue_cores:27``; ``core/context/build_context.py``
``CPU_AFFINITY`` handling ``:367-393``; ``msrun --bind_core``). On a GPU host the useful split is by NUMA node: a rank
gets an equal slice of the cores of the NUMA node its GPU hangs off (from sysfs), minus cores the caller reserves.
Everything is read-only with respect to the GPU: only ``os.sched_setaffinity`` of the calling process is changed.
"""
from __future__ import annotations

import glob
import os
import re
from typing import Dict, Iterable, List, Optional

from .bit_array import BitArray


def parse_cpu_list(text: str) -> List[int]:
    """``"0-3,8,10-11"`` → ``[0, 1, 2, 3, 8, 10, 11]``."""
    out: List[int] = []
    for part in text.strip().split(","):
        part = part.strip()
        if not part:
            continue
        if "-" in part:
            a, b = part.split("-", 1)
            out.extend(range(int(a), int(b) + 1))
        else:
            out.append(int(part))
    return sorted(set(out))


def format_cpu_list(cpus: Iterable[int]) -> str:
    cpus = sorted(set(cpus))
    parts, i = [], 0
    while i < len(cpus):
        j = i
        while j + 1 < len(cpus) and cpus[j + 1] == cpus[j] + 1:
            j += 1
        parts.append(str(cpus[i]) if i == j else f"{cpus[i]}-{cpus[j]}")
        i = j + 1
    return ",".join(parts)


def numa_nodes(sys_root: str = "/sys/devices/system/node") -> Dict[int, List[int]]:
    """NUMA node → CPU list from sysfs (empty when the host does not expose it)."""
    nodes: Dict[int, List[int]] = {}
    for path in glob.glob(os.path.join(sys_root, "node[0-9]*")):
        m = re.search(r"node(\d+)$", path)
        try:
            with open(os.path.join(path, "cpulist")) as f:
                nodes[int(m.group(1))] = parse_cpu_list(f.read())
        except OSError:
            continue
    return nodes


def gpu_numa_node(pci_bus_id: str, sys_root: str = "/sys/bus/pci/devices") -> Optional[int]:
    """NUMA node of a PCI device (``0000:1b:00.0``), or None if sysfs does not say (value -1)."""
    try:
        with open(os.path.join(sys_root, pci_bus_id.lower(), "numa_node")) as f:
            node = int(f.read().strip())
        return node if node >= 0 else None
    except (OSError, ValueError):
        return None


def cores_for_rank(local_rank: int, local_world: int, available: Iterable[int], reserved: Iterable[int] = (),
                   numa: Optional[Dict[int, List[int]]] = None, gpu_node: Optional[int] = None) -> List[int]:
    """Cores for one rank: the rank's share of its GPU's NUMA node when known (ranks of the same node split it in
    order), else an equal contiguous slice of all available cores. ``reserved`` cores are never handed out."""
    usable = BitArray.from_indices(available) - BitArray.from_indices(reserved)
    cpus = usable.get_marked_index()
    if not cpus:
        raise ValueError("no CPU cores left after removing the reserved ones")
    if numa and gpu_node is not None and gpu_node in numa:
        node_cpus = [c for c in numa[gpu_node] if usable.get(c)]
        ranks_per_node = max(1, local_world // max(1, len(numa)))
        pos = local_rank % ranks_per_node
        per = max(1, len(node_cpus) // ranks_per_node)
        share = node_cpus[pos * per:(pos + 1) * per]
        if share:
            return share
    per = max(1, len(cpus) // max(1, local_world))
    share = cpus[local_rank * per:(local_rank + 1) * per]
    return share or cpus


def bind_rank_to_cores(local_rank: Optional[int] = None, local_world: Optional[int] = None,
                       affinity_cpu_list: Optional[Dict[str, str]] = None, reserved: Iterable[int] = ()) -> List[int]:
    """Apply the split to the calling process and return the cores. ``affinity_cpu_list`` (YAML
    ``context.affinity_cpu_list``: ``{"device0": "0-15", …}``) overrides the automatic choice."""
    local_rank = int(os.environ.get("LOCAL_RANK", "0")) if local_rank is None else local_rank
    local_world = int(os.environ.get("LOCAL_WORLD_SIZE", "1")) if local_world is None else local_world
    available = sorted(os.sched_getaffinity(0))
    if affinity_cpu_list and f"device{local_rank}" in affinity_cpu_list:
        cores = [c for c in parse_cpu_list(affinity_cpu_list[f"device{local_rank}"]) if c in set(available)]
    else:
        node = None
        try:
            import torch
            if torch.cuda.is_available():
                bus = torch.cuda.get_device_properties(local_rank).pci_bus_id
                dom = getattr(torch.cuda.get_device_properties(local_rank), "pci_domain_id", 0)
                dev = torch.cuda.get_device_properties(local_rank).pci_device_id
                node = gpu_numa_node(f"{dom:04x}:{bus:02x}:{dev:02x}.0")
        except Exception:       # the topology is a hint; without it the equal split applies
            node = None
        cores = cores_for_rank(local_rank, local_world, available, reserved, numa_nodes(), node)
    if cores:
        os.sched_setaffinity(0, cores)
    return cores
