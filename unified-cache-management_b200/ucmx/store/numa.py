"""Keep a process (and therefore the pages it page-locks) on the NUMA node its GPU hangs off.

Page-locked staging memory is placed by first touch: an unbound process may put it on the other
socket, and every byte of an offload then crosses the inter-socket link as well as PCIe.  The
reference pins its retrieval threads per NUMA node for the same reason
(ucm/sparse/kvstar/retrieve/core/api/kvstar_retrieve/kvstar_retrieve.cpp, SetupParam.perNumaCoreIds).
Everything here reads sysfs only; when a file is missing the call does nothing and says so.
"""
from __future__ import annotations

import os
from typing import List, Optional


def _parse_cpulist(text: str) -> List[int]:
    cpus: List[int] = []
    for part in text.strip().split(","):
        if not part:
            continue
        if "-" in part:
            lo, hi = part.split("-")
            cpus.extend(range(int(lo), int(hi) + 1))
        else:
            cpus.append(int(part))
    return cpus


def device_numa_node(pci_bus_id: str, sysfs: str = "/sys") -> Optional[int]:
    """NUMA node of a PCI device given as 'dddd:bb:dd.f' (any case), or None when sysfs does not say."""
    try:
        with open(os.path.join(sysfs, "bus", "pci", "devices", pci_bus_id.lower(), "numa_node")) as f:
            node = int(f.read().strip())
        return node if node >= 0 else None
    except (OSError, ValueError):
        return None


def node_cpus(node: int, sysfs: str = "/sys") -> List[int]:
    try:
        with open(os.path.join(sysfs, "devices", "system", "node", f"node{node}", "cpulist")) as f:
            return _parse_cpulist(f.read())
    except (OSError, ValueError):
        return []


def bind_to_device_node(device_index: int, sysfs: str = "/sys") -> Optional[int]:
    """Restrict this process to the CPUs of the NUMA node of CUDA device `device_index`.
    Returns the node, or None when it could not be determined (nothing is changed then)."""
    import torch
    props = torch.cuda.get_device_properties(device_index)
    bus_id = getattr(props, "pci_bus_id", None)
    if isinstance(bus_id, int) or bus_id is None:      # older torch: numeric fields only
        domain = getattr(props, "pci_domain_id", 0)
        bus_id = f"{domain:04x}:{getattr(props, 'pci_bus_id', 0):02x}:{getattr(props, 'pci_device_id', 0):02x}.0"
    node = device_numa_node(str(bus_id), sysfs)
    if node is None:
        return None
    cpus = [c for c in node_cpus(node, sysfs) if c in os.sched_getaffinity(0)]
    if not cpus:
        return None
    os.sched_setaffinity(0, cpus)
    return node
