"""CPU / NUMA placement of a rank process next to its GPU.

The reference pins worker threads to cores and checks that tensors live on the worker's NUMA node
(native/src/main/c/simd/vector_runtime.c:25-191: ``runtime_numa_node_of_cpu`` from sysfs, ``runtime_pin_current_thread`` via
``sched_setaffinity``; tensor/.../tensorlib/TensorRuntime.java:77-99 ANALYZE / ENFORCE modes). With one process per GPU the
equivalent is done once at launch: find the NUMA node the GPU's PCI function hangs off, and restrict the process (host-side
scheduler, tokenizer, pinned staging buffers, NCCL proxy threads) to that node's cores, so host->device copies and launch
latency do not cross the socket interconnect.

Modes (env ``DLV_AFFINITY`` or the ``mode`` argument): ``off``; ``analyze`` (report only); ``enforce`` (default when called):
set the affinity. Everything is read from sysfs; ``sysfs_root`` exists so tests can point at a fake tree.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Optional


def parse_cpulist(text: str) -> list:
    """``"0-3,8,10-11"`` -> [0, 1, 2, 3, 8, 10, 11]."""
    cpus: list = []
    for part in text.strip().split(","):
        if not part:
            continue
        if "-" in part:
            a, b = part.split("-")
            cpus.extend(range(int(a), int(b) + 1))
        else:
            cpus.append(int(part))
    return cpus


def normalise_pci_bus_id(bus_id: str) -> str:
    """CUDA reports ``00000000:1B:00.0`` (8-digit domain, upper case); sysfs names it ``0000:1b:00.0``."""
    parts = bus_id.strip().lower().split(":")
    if len(parts) == 3:
        parts[0] = parts[0][-4:].rjust(4, "0")
    elif len(parts) == 2:
        parts = ["0000"] + parts
    return ":".join(parts)


@dataclass
class Placement:
    device: int
    pci_bus_id: str = ""
    numa_node: int = -1
    cpus: list = field(default_factory=list)
    applied: bool = False
    note: str = ""

    def to_json(self) -> dict:
        return {"device": self.device, "pci_bus_id": self.pci_bus_id, "numa_node": self.numa_node, "cpus": len(self.cpus), "applied": self.applied,
                "note": self.note}


def gpu_numa_node(pci_bus_id: str, sysfs_root: str = "/sys") -> int:
    p = os.path.join(sysfs_root, "bus", "pci", "devices", normalise_pci_bus_id(pci_bus_id), "numa_node")
    try:
        with open(p) as f:
            return int(f.read().strip())
    except (OSError, ValueError):
        return -1


def node_cpus(node: int, sysfs_root: str = "/sys") -> list:
    try:
        with open(os.path.join(sysfs_root, "devices", "system", "node", f"node{node}", "cpulist")) as f:
            return parse_cpulist(f.read())
    except OSError:
        return []


def numa_node_of_cpu(cpu: int, sysfs_root: str = "/sys") -> int:
    d = os.path.join(sysfs_root, "devices", "system", "cpu", f"cpu{cpu}")
    try:
        for name in os.listdir(d):
            if name.startswith("node") and name[4:].isdigit():
                return int(name[4:])
    except OSError:
        pass
    return -1


def split_among_local_ranks(cpus: list, ranks_on_node: int, index: int) -> list:
    """Several GPUs usually share a NUMA node: give each of their processes a contiguous share of the node's cores."""
    if ranks_on_node <= 1 or len(cpus) < ranks_on_node:
        return list(cpus)
    per = len(cpus) // ranks_on_node
    return cpus[index * per : (index + 1) * per]


def place_rank(device: int, pci_bus_id: Optional[str] = None, mode: Optional[str] = None, sysfs_root: str = "/sys", ranks_on_node: int = 1,
               index_on_node: int = 0, setaffinity=os.sched_setaffinity, allowed: Optional[set] = None) -> Placement:
    """Pin this process to the cores of the NUMA node of GPU ``device``. Never raises: a machine without the sysfs entries
    (containers, single-socket boxes reporting node -1) is left as it is and the reason is recorded in ``note``."""
    mode = (mode or os.environ.get("DLV_AFFINITY", "enforce")).lower()
    pl = Placement(device)
    if mode == "off":
        pl.note = "off"
        return pl
    if pci_bus_id is None:
        try:
            import torch

            pci_bus_id = torch.cuda.get_device_properties(device).pci_bus_id  # type: ignore[attr-defined]
            pci_bus_id = pci_bus_id if isinstance(pci_bus_id, str) else f"0000:{int(pci_bus_id):02x}:00.0"
        except Exception as e:  # noqa: BLE001 - no CUDA device: nothing to place
            pl.note = f"no PCI id for device {device}: {e}"
            return pl
    pl.pci_bus_id = normalise_pci_bus_id(pci_bus_id)
    pl.numa_node = gpu_numa_node(pl.pci_bus_id, sysfs_root)
    if pl.numa_node < 0:
        pl.note = "the GPU reports no NUMA node"
        return pl
    cpus = node_cpus(pl.numa_node, sysfs_root)
    allowed = set(os.sched_getaffinity(0)) if allowed is None else allowed
    cpus = [c for c in cpus if c in allowed]
    pl.cpus = split_among_local_ranks(cpus, ranks_on_node, index_on_node)
    if not pl.cpus:
        pl.note = f"no usable cores on node {pl.numa_node}"
        return pl
    if mode == "analyze":
        pl.note = "analyze only"
        return pl
    try:
        setaffinity(0, set(pl.cpus))
        pl.applied = True
    except OSError as e:
        pl.note = f"sched_setaffinity failed: {e}"
    return pl


def place_local_rank(local_rank: int, local_world: int, mode: Optional[str] = None, sysfs_root: str = "/sys", bus_ids: Optional[list] = None,
                     **kw) -> Placement:
    """``place_rank`` for rank ``local_rank`` of ``local_world`` processes that use GPUs 0..local_world-1 of this machine: the
    node's cores are divided among the ranks whose GPUs sit on the same node."""
    if bus_ids is None:
        try:
            import torch

            bus_ids = [torch.cuda.get_device_properties(i).pci_bus_id for i in range(local_world)]  # type: ignore[attr-defined]
        except Exception:  # noqa: BLE001
            return place_rank(local_rank, None, mode, sysfs_root, **kw)
    nodes = [gpu_numa_node(b, sysfs_root) for b in bus_ids]
    mine = nodes[local_rank]
    same = [i for i, n in enumerate(nodes) if n == mine]
    return place_rank(local_rank, bus_ids[local_rank], mode, sysfs_root, ranks_on_node=len(same), index_on_node=same.index(local_rank), **kw)
