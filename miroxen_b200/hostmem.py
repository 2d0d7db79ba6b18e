"""Host-side placement for the host-buffer entry points (mxk_dit_block_ops_host).

A block that comes from host memory is bound by the PCIe path between the pinned buffers and the GPU.  On a
two-socket host a rank whose pinned buffers sit on the other socket's memory pulls every byte across the
socket interconnect, and several ranks doing so share that one link.  `bind_to_device_node` moves the calling
process onto the CPUs of the NUMA node the GPU's PCIe root belongs to BEFORE it allocates its pinned buffers,
so that first-touch placement puts them next to the GPU.  It reads sysfs only and changes nothing but this
process's own CPU affinity; where the host reports no NUMA node for the device (a single-node or virtualised
host) it does nothing and says so.
"""
from __future__ import annotations

import os
from pathlib import Path

SYSFS = Path("/sys")


def parse_cpulist(text: str) -> list[int]:
    """'0-3,8,10-11' -> [0, 1, 2, 3, 8, 10, 11] (the format of sysfs cpulist files)."""
    cpus: list[int] = []
    for part in text.strip().split(","):
        if not part:
            continue
        if "-" in part:
            lo, hi = part.split("-")
            cpus.extend(range(int(lo), int(hi) + 1))
        else:
            cpus.append(int(part))
    return cpus


def pci_address(domain: int, bus: int, device: int) -> str:
    """sysfs name of function 0 of a PCI device."""
    return f"{domain:04x}:{bus:02x}:{device:02x}.0"


def device_numa_node(pci_addr: str, sysfs: Path = SYSFS) -> int | None:
    """NUMA node of a PCI device, or None when sysfs has no answer (file absent or -1)."""
    f = sysfs / "bus" / "pci" / "devices" / pci_addr / "numa_node"
    try:
        node = int(f.read_text().strip())
    except (OSError, ValueError):
        return None
    return node if node >= 0 else None


def node_cpus(node: int, sysfs: Path = SYSFS) -> list[int]:
    f = sysfs / "devices" / "system" / "node" / f"node{node}" / "cpulist"
    try:
        return parse_cpulist(f.read_text())
    except (OSError, ValueError):
        return []


def plan_binding(pci_addr: str, allowed: set[int], sysfs: Path = SYSFS) -> dict:
    """What bind_to_device_node would do: {"node": n | None, "cpus": [...], "why": "..."}.
    `allowed` is the CPU set the process may run on now (a cgroup or an outer taskset may have narrowed it);
    the binding never widens it."""
    node = device_numa_node(pci_addr, sysfs)
    if node is None:
        return {"node": None, "cpus": [], "why": f"no NUMA node reported for {pci_addr}"}
    cpus = sorted(set(node_cpus(node, sysfs)) & allowed)
    if not cpus:
        return {"node": node, "cpus": [], "why": f"none of node {node}'s CPUs is available to this process"}
    return {"node": node, "cpus": cpus, "why": "bound"}


def bind_to_device_node(device_index: int, sysfs: Path = SYSFS) -> dict:
    """Restrict this process to the CPUs of the NUMA node of CUDA device `device_index`.  Call it before the
    pinned host buffers are allocated.  Returns the plan (see plan_binding); never raises for a host that
    cannot answer."""
    import torch
    try:
        p = torch.cuda.get_device_properties(device_index)
        addr = pci_address(p.pci_domain_id, p.pci_bus_id, p.pci_device_id)
    except (AttributeError, RuntimeError) as e:
        return {"node": None, "cpus": [], "why": f"no PCI address for device {device_index}: {e}"}
    plan = plan_binding(addr, set(os.sched_getaffinity(0)), sysfs)
    plan["pci"] = addr
    if plan["cpus"]:
        try:
            os.sched_setaffinity(0, plan["cpus"])
        except OSError as e:
            plan["why"], plan["cpus"] = f"sched_setaffinity refused: {e}", []
    return plan
