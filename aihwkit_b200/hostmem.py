"""Host-side placement for the page-locked buffers that feed a GPU.

A GPU reads page-locked host memory over PCIe through the CPU socket it is attached to.  Memory
that the allocating thread first touched on the other socket crosses the inter-socket link on
every copy, and with one process per GPU all of them then share that link.  Binding the process
to the CPUs next to its GPU before it allocates keeps every rank's staging buffers on its own
socket (first-touch placement)."""

from __future__ import annotations

import os
from typing import Optional, Set


def _parse_cpulist(text: str) -> Set[int]:
    cpus: Set[int] = set()
    for part in text.strip().split(","):
        if not part:
            continue
        if "-" in part:
            lo, hi = part.split("-")
            cpus.update(range(int(lo), int(hi) + 1))
        else:
            cpus.add(int(part))
    return cpus


def gpu_local_cpus(device_index: int) -> Optional[Set[int]]:
    """CPUs of the NUMA node the GPU's PCIe slot belongs to, from sysfs; ``None`` if unknown."""
    try:
        import torch

        prop = torch.cuda.get_device_properties(device_index)
        bus = f"{prop.pci_domain_id:04x}:{prop.pci_bus_id:02x}:{prop.pci_device_id:02x}.0"
        with open(f"/sys/bus/pci/devices/{bus}/local_cpulist", "r", encoding="ascii") as f:
            cpus = _parse_cpulist(f.read())
        return cpus or None
    except (OSError, AttributeError, ValueError, RuntimeError):
        return None


def bind_to_gpu_numa(device_index: int) -> Optional[int]:
    """Restrict this process to the CPUs next to ``device_index`` (intersected with the CPUs it
    may already use).  Call it before allocating page-locked memory.  Returns the number of CPUs
    the process is bound to, or ``None`` when the topology is unknown or the call is not
    permitted (nothing changes then)."""
    cpus = gpu_local_cpus(device_index)
    if not cpus:
        return None
    try:
        allowed = os.sched_getaffinity(0)
        target = (cpus & allowed) or None
        if target is None:
            return None
        os.sched_setaffinity(0, target)
        return len(target)
    except (OSError, AttributeError):
        return None
