"""CPU / memory affinity: bind a worker process to the NUMA node closest to its GPU (libnuma through ctypes, the
approach of nemo_rl/distributed/numa_utils.py:39). Silently does nothing when libnuma or the sysfs entries are absent."""

from __future__ import annotations

import ctypes
import ctypes.util
import os
from typing import Optional


def gpu_numa_node(gpu_index: int) -> Optional[int]:
    """NUMA node of a GPU from its PCI bus id (``/sys/bus/pci/devices/<bus>/numa_node``)."""
    try:
        import pynvml

        pynvml.nvmlInit()
        try:   # a process-local CUDA ordinal maps to the NVML index through CUDA_VISIBLE_DEVICES (numeric entries)
            from rl_b200.utils.nvml import device_id_to_physical

            phys = device_id_to_physical(gpu_index)
            if 0 <= phys < pynvml.nvmlDeviceGetCount():
                gpu_index = phys
        except Exception:
            pass
        h = pynvml.nvmlDeviceGetHandleByIndex(gpu_index)
        bus = pynvml.nvmlDeviceGetPciInfo(h).busId
        bus = bus.decode() if isinstance(bus, bytes) else bus
        path = f"/sys/bus/pci/devices/{bus.lower()[-12:]}/numa_node"
        if os.path.exists(path):
            node = int(open(path).read().strip())
            return node if node >= 0 else None
    except Exception:
        return None
    return None


def bind_to_node(node: int) -> bool:
    name = ctypes.util.find_library("numa")
    if not name:
        return False
    lib = ctypes.CDLL(name)
    if lib.numa_available() < 0:
        return False
    lib.numa_run_on_node(ctypes.c_int(node))
    lib.numa_set_preferred(ctypes.c_int(node))
    return True


def bind_to_gpu_numa_node(gpu_index: int) -> bool:
    node = gpu_numa_node(gpu_index)
    return bind_to_node(node) if node is not None else False
