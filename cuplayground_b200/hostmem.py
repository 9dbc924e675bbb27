"""Host-side placement for the host-activation path (aristos_moe_submit_host): run the calling thread on the CPUs of
the NUMA node the GPU hangs off, so that pinned staging buffers allocated afterwards (first touch) and the copy
submissions are local to the GPU's PCIe root. Reads sysfs only; nothing on the GPU is queried beyond its PCI address
and nothing is set on it."""
from __future__ import annotations

import os
from typing import Optional


def _parse_cpulist(text: str) -> set[int]:
    cpus: set[int] = set()
    for part in text.strip().split(","):
        if not part:
            continue
        lo, _, hi = part.partition("-")
        cpus.update(range(int(lo), int(hi or lo) + 1))
    return cpus


def gpu_numa_node(device_index: int, sysfs: str = "/sys") -> Optional[int]:
    """NUMA node of a CUDA device from /sys/bus/pci/devices/<bdf>/numa_node; None when it cannot be read or the
    platform reports -1."""
    import torch
    p = torch.cuda.get_device_properties(device_index)
    try:
        bdf = f"{p.pci_domain_id:04x}:{p.pci_bus_id:02x}:{p.pci_device_id:02x}.0"
    except AttributeError:
        return None
    try:
        with open(os.path.join(sysfs, "bus/pci/devices", bdf, "numa_node")) as f:
            node = int(f.read().strip())
    except (OSError, ValueError):
        return None
    return node if node >= 0 else None


def node_cpus(node: int, sysfs: str = "/sys") -> set[int]:
    try:
        with open(os.path.join(sysfs, "devices/system/node", f"node{node}", "cpulist")) as f:
            return _parse_cpulist(f.read())
    except OSError:
        return set()


def plan_binding(allowed: set[int], node: Optional[int], cpus_of_node: set[int]) -> Optional[set[int]]:
    """The CPU set to run on: the allowed CPUs that belong to the GPU's node, or None to leave the affinity alone
    (unknown node, or none of the node's CPUs is allowed to this process)."""
    if node is None:
        return None
    local = allowed & cpus_of_node
    return local if local and local != allowed else None


def bind_to_gpu_numa_node(device_index: int, sysfs: str = "/sys") -> dict:
    """Restrict the calling thread to the CPUs of the GPU's NUMA node when that narrows its affinity. Returns what
    was found and done (for the benchmark's record)."""
    try:
        allowed = set(os.sched_getaffinity(0))
    except AttributeError:
        return {"gpu_node": None, "bound": False, "reason": "no sched_getaffinity on this platform"}
    node = gpu_numa_node(device_index, sysfs)
    cpus = node_cpus(node, sysfs) if node is not None else set()
    target = plan_binding(allowed, node, cpus)
    info = {"gpu_node": node, "cpus_allowed": len(allowed), "cpus_on_gpu_node": len(allowed & cpus), "bound": False}
    if target is not None:
        try:
            os.sched_setaffinity(0, target)
            info["bound"] = True
        except OSError as e:
            info["reason"] = repr(e)
    elif node is not None and allowed and allowed <= cpus:
        info["reason"] = "every allowed CPU is already on the GPU's node"
    return info
