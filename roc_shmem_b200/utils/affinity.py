"""CPU / memory placement next to a GPU.

Pinned host buffers land on the NUMA node of the thread that first touches them; when eight ranks of a node stage their
inputs through pinned memory, buffers on the wrong socket cross the inter-socket link before they reach the GPU's PCIe
root.  `bind_to_gpu(device)` restricts the calling process to the CPUs the kernel lists as local to that GPU
(`/sys/bus/pci/devices/<bus id>/local_cpulist`), so later pinned allocations are node-local.  It changes nothing about
the GPU itself and is a no-op when the topology files are not there.
"""
from __future__ import annotations

import os
from pathlib import Path
from typing import Optional


def _parse_cpulist(text: str) -> set[int]:
    cpus: set[int] = set()
    for part in text.strip().split(","):
        if not part:
            continue
        if "-" in part:
            a, b = part.split("-")
            cpus.update(range(int(a), int(b) + 1))
        else:
            cpus.add(int(part))
    return cpus


def local_cpus(device: int, sysfs: str = "/sys/bus/pci/devices") -> Optional[set[int]]:
    """CPUs local to CUDA device `device`, or None if unknown."""
    try:
        import torch
        p = torch.cuda.get_device_properties(device)
        bus = f"{p.pci_domain_id:04x}:{p.pci_bus_id:02x}:{p.pci_device_id:02x}.0"
        text = (Path(sysfs) / bus / "local_cpulist").read_text()
    except Exception:
        return None
    cpus = _parse_cpulist(text)
    return cpus or None


def bind_to_gpu(device: int) -> Optional[set[int]]:
    """Restrict this process to the CPUs local to the GPU (intersected with what it may already use).  Returns the
    CPU set in effect, or None if nothing was changed."""
    cpus = local_cpus(device)
    if not cpus or not hasattr(os, "sched_setaffinity"):
        return None
    allowed = os.sched_getaffinity(0) & cpus
    if not allowed:
        return None
    try:
        os.sched_setaffinity(0, allowed)
    except OSError:
        return None
    return allowed
