"""Read-only sampling of SM clocks and throttle reasons while a timed region runs (NVML)."""
from __future__ import annotations

import statistics
import threading
import time


class ClockSampler:
    """Background thread polling NVML every ``period_s``; never changes any GPU setting."""

    _REASONS = {
        0x0000000000000004: "sw_power_cap",
        0x0000000000000008: "hw_slowdown",
        0x0000000000000020: "sw_thermal_slowdown",
        0x0000000000000040: "hw_thermal_slowdown",
        0x0000000000000080: "hw_power_brake_slowdown",
    }

    def __init__(self, device_index: int = 0, period_s: float = 0.1):
        self.idx, self.period = device_index, period_s
        self.samples, self.reasons, self.power = [], set(), []
        self.max_mhz = None
        self._stop = threading.Event()
        self._thr = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = self._handle_of(pynvml, device_index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nv = None

    @staticmethod
    def _handle_of(nv, cuda_index: int):
        """NVML handle of the CUDA device ``cuda_index``. CUDA ordinals follow CUDA_VISIBLE_DEVICES,
        NVML indices do not, so the device is looked up by its UUID (falling back to the PCI bus id,
        then to the plain index when torch is not importable)."""
        try:
            import torch

            props = torch.cuda.get_device_properties(cuda_index)
            uuid = getattr(props, "uuid", None)
            if uuid is not None:
                try:
                    return nv.nvmlDeviceGetHandleByUUID(("GPU-" + str(uuid)).encode())
                except Exception:
                    pass
            bus = "%08x:%02x:%02x.0" % (getattr(props, "pci_domain_id", 0), props.pci_bus_id,
                                        props.pci_device_id)
            return nv.nvmlDeviceGetHandleByPciBusId(bus.encode())
        except Exception:
            return nv.nvmlDeviceGetHandleByIndex(cuda_index)

    def _loop(self):
        nv = self._nv
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self._h) if hasattr(
                    nv, "nvmlDeviceGetCurrentClocksEventReasons") else nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)
                for bit, name in self._REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
                self.power.append(nv.nvmlDeviceGetPowerUsage(self._h) / 1000.0)
            except Exception:
                pass
            time.sleep(self.period)

    def start(self):
        if self._nv is not None:
            self._thr = threading.Thread(target=self._loop, daemon=True)
            self._thr.start()
        return self

    def stop(self) -> dict:
        self._stop.set()
        if self._thr is not None:
            self._thr.join(timeout=2)
        return self.summary()

    def summary(self) -> dict:
        return {
            "sm_mhz": statistics.median(self.samples) if self.samples else None,
            "sm_max_mhz": self.max_mhz,
            "reasons": sorted(self.reasons),
            "power_w_max": max(self.power) if self.power else None,
            "samples": len(self.samples),
        }
