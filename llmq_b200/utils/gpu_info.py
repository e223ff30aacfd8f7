"""GPU telemetry through NVML (read-only) with a torch-only fallback.

Mirrors IGPUUtilTracker / GPUUtilInfo of the reference (src/utilities/gpu_info.h:40-47, gpu_info_nvml.cpp:127-252):
clock, power (from the energy counter when available), temperature, fan, throttle reasons, utilisation, free
memory and PCIe throughput.  Nothing here changes a GPU setting.
"""
from __future__ import annotations

import os
import time
from dataclasses import asdict, dataclass

import torch


@dataclass
class GPUUtilInfo:
    clock: int = 0
    max_clock: int = 0
    fan: int = 0
    power: int = 0              # mW
    power_limit: int = 0        # mW
    temperature: int = 0
    temp_slowdown: int = 0
    gpu_utilization: int = 0
    mem_utilization: int = 0
    throttle_reason: str = ""
    mem_free: int = 0
    mem_total: int = 0
    mem_reserved: int = 0
    pcie_rx: int = 0
    pcie_tx: int = 0

    def to_dict(self):
        return asdict(self)


_THROTTLE_BITS = [(0x1, "gpu_idle"), (0x2, "app_clocks"), (0x4, "sw_power_cap"), (0x8, "hw_slowdown"), (0x10, "sync_boost"),
                  (0x20, "sw_thermal_slowdown"), (0x40, "hw_thermal_slowdown"), (0x80, "hw_power_brake"), (0x100, "display_clocks")]


def _nvml():
    try:
        import pynvml
        pynvml.nvmlInit()
        return pynvml
    except Exception:
        return None


class GPUUtilTracker:
    def __init__(self, device_index: int = 0, nvml=None):
        """``nvml`` may be an object with the pynvml function names (used by the CPU tests with a fake)."""
        self.index = device_index
        self.nvml = nvml if nvml is not None else _nvml()
        self.handle = None
        self._last_energy = None
        if self.nvml is not None:
            try:
                self.handle = self.nvml.nvmlDeviceGetHandleByIndex(self._physical_index(device_index))
            except Exception:
                self.handle = None

    @staticmethod
    def _physical_index(i: int) -> int:
        vis = os.environ.get("CUDA_VISIBLE_DEVICES")
        if vis:
            parts = [p for p in vis.split(",") if p.strip() != ""]
            if i < len(parts) and parts[i].strip().isdigit():
                return int(parts[i])
        return i

    def _try(self, fn, *a, default=0):
        try:
            return fn(self.handle, *a)
        except Exception:
            return default

    def update(self) -> GPUUtilInfo:
        info = GPUUtilInfo()
        n, h = self.nvml, self.handle
        if n is None or h is None:
            if torch.cuda.is_available():
                free, total = torch.cuda.mem_get_info(self.index)
                info.mem_free, info.mem_total = free, total
                info.mem_reserved = torch.cuda.memory_reserved(self.index)
            return info
        info.clock = self._try(n.nvmlDeviceGetClockInfo, getattr(n, "NVML_CLOCK_SM", 1))
        info.max_clock = self._try(n.nvmlDeviceGetMaxClockInfo, getattr(n, "NVML_CLOCK_SM", 1))
        info.fan = self._try(n.nvmlDeviceGetFanSpeed)
        now = time.monotonic()
        energy = self._try(n.nvmlDeviceGetTotalEnergyConsumption, default=None)      # mJ
        if energy is not None and self._last_energy is not None and now > self._last_energy[1]:
            info.power = int((energy - self._last_energy[0]) / (now - self._last_energy[1]))
        else:
            info.power = self._try(n.nvmlDeviceGetPowerUsage)
        if energy is not None:
            self._last_energy = (energy, now)
        info.power_limit = self._try(n.nvmlDeviceGetEnforcedPowerLimit)
        info.temperature = self._try(n.nvmlDeviceGetTemperature, getattr(n, "NVML_TEMPERATURE_GPU", 0))
        info.temp_slowdown = self._try(n.nvmlDeviceGetTemperatureThreshold, getattr(n, "NVML_TEMPERATURE_THRESHOLD_SLOWDOWN", 1))
        util = self._try(n.nvmlDeviceGetUtilizationRates, default=None)
        if util is not None:
            info.gpu_utilization, info.mem_utilization = int(util.gpu), int(util.memory)
        reasons = self._try(n.nvmlDeviceGetCurrentClocksEventReasons, default=None)
        if reasons is None:
            reasons = self._try(n.nvmlDeviceGetCurrentClocksThrottleReasons, default=0)
        info.throttle_reason = "|".join(name for bit, name in _THROTTLE_BITS if reasons & bit and name != "gpu_idle") or "none"
        mem = self._try(n.nvmlDeviceGetMemoryInfo, default=None)
        if mem is not None:
            info.mem_free, info.mem_total = int(mem.free), int(mem.total)
        info.pcie_rx = self._try(n.nvmlDeviceGetPcieThroughput, getattr(n, "NVML_PCIE_UTIL_RX_BYTES", 1))
        info.pcie_tx = self._try(n.nvmlDeviceGetPcieThroughput, getattr(n, "NVML_PCIE_UTIL_TX_BYTES", 0))
        if torch.cuda.is_available():
            info.mem_reserved = torch.cuda.memory_reserved(self.index)
        return info


def get_gpu_name(index: int = 0) -> str:
    return torch.cuda.get_device_name(index) if torch.cuda.is_available() else "cpu"


def set_cpu_affinity(device_index: int, nvml=None) -> bool:
    """Pins the calling thread to the CPUs NVML reports as close to the GPU; returns False when unavailable."""
    n = nvml if nvml is not None else _nvml()
    if n is None:
        return False
    try:
        h = n.nvmlDeviceGetHandleByIndex(GPUUtilTracker._physical_index(device_index))
        words = n.nvmlDeviceGetCpuAffinity(h, (os.cpu_count() + 63) // 64)
        cpus = {w * 64 + b for w, word in enumerate(words) for b in range(64) if word >> b & 1}
        cpus &= set(os.sched_getaffinity(0))
        if cpus:
            os.sched_setaffinity(0, cpus)
            return True
    except Exception:
        pass
    return False
