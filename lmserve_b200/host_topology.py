"""Where a GPU sits in the host: its PCIe link, its NUMA node and the CPU cores next to it.

LMServe binds each worker process to the cores that are local to its GPU before it allocates
its pinned pools (``runtime/worker/llm_worker/utils.py:51-80``: ``nvidia-smi`` for the PCI
address, then ``/sys/class/pci_bus/<bus>/cpuaffinity``), so that the host side of every
GPU<->host copy stays on the GPU's own socket.  The same here, from the PCI address CUDA
reports and sysfs alone; every function returns ``None`` / does nothing when sysfs has no
answer (containers often hide it).  Read-only: nothing here changes a device setting.
"""
from __future__ import annotations

import os
from pathlib import Path
from typing import Dict, List, Optional

import torch


def pci_address(device_index: int) -> Optional[str]:
    """``dddd:bb:dd.0`` of a CUDA device."""
    try:
        p = torch.cuda.get_device_properties(device_index)
        return f"{p.pci_domain_id:04x}:{p.pci_bus_id:02x}:{p.pci_device_id:02x}.0"
    except Exception:  # noqa: BLE001 - older torch without the PCI fields, or no device
        return None


def _read(path: Path) -> Optional[str]:
    try:
        return path.read_text().strip()
    except OSError:
        return None


def parse_cpu_list(text: str) -> List[int]:
    """``"0-3,8,10-11"`` -> ``[0, 1, 2, 3, 8, 10, 11]`` (the format of ``local_cpulist``)."""
    cpus: List[int] = []
    for part in text.split(","):
        part = part.strip()
        if not part:
            continue
        if "-" in part:
            a, b = part.split("-")
            cpus.extend(range(int(a), int(b) + 1))
        else:
            cpus.append(int(part))
    return cpus


def pcie_link(device_index: int, sysfs: str = "/sys/bus/pci/devices") -> Dict[str, Optional[str]]:
    """Negotiated and maximum PCIe link of the GPU, NUMA node and local CPU list, as sysfs
    states them (``current_link_speed`` reads like ``32.0 GT/s PCIe`` for Gen5)."""
    addr = pci_address(device_index)
    out: Dict[str, Optional[str]] = {"pci_address": addr}
    if addr is None:
        return out
    base = Path(sysfs) / addr
    for key in ("current_link_speed", "current_link_width", "max_link_speed", "max_link_width",
                "numa_node", "local_cpulist"):
        out[key] = _read(base / key)
    if out["current_link_speed"] is None:
        out.update(_nvml_link(device_index))     # containers often hide the sysfs attributes
    return out


def _nvml_link(device_index: int) -> Dict[str, Optional[str]]:
    """The same link facts through NVML queries (read-only), where sysfs does not show them."""
    try:
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(device_index)
        return {"current_link_gen": str(pynvml.nvmlDeviceGetCurrPcieLinkGeneration(h)),
                "current_link_width": str(pynvml.nvmlDeviceGetCurrPcieLinkWidth(h)),
                "max_link_gen": str(pynvml.nvmlDeviceGetMaxPcieLinkGeneration(h)),
                "max_link_width": str(pynvml.nvmlDeviceGetMaxPcieLinkWidth(h)),
                "source": "nvml"}
    except Exception:  # noqa: BLE001 - no NVML, no answer
        return {}


def local_cpus(device_index: int, sysfs: str = "/sys/bus/pci/devices") -> Optional[List[int]]:
    text = pcie_link(device_index, sysfs).get("local_cpulist")
    if not text:
        return None
    try:
        return parse_cpu_list(text) or None
    except ValueError:
        return None


def set_cpu_affinity_for_gpu(device_index: int, sysfs: str = "/sys/bus/pci/devices") -> Optional[List[int]]:
    """Binds the calling process to the cores local to the GPU (the role of
    ``set_cpu_affinity_for_gpu``, ``utils.py:51-80``); call it before pinned pools are
    allocated.  Returns the cores it bound to, or ``None`` when it left the affinity alone."""
    cpus = local_cpus(device_index, sysfs)
    if not cpus:
        return None
    try:
        allowed = os.sched_getaffinity(0)
        want = sorted(set(cpus) & set(allowed))
        if not want:
            return None
        os.sched_setaffinity(0, want)
        return want
    except (AttributeError, OSError):
        return None
