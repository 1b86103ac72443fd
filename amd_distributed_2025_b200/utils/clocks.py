"""Read-only sampling of SM clocks, power and throttle reasons while a benchmark runs.

A background thread polls NVML every few milliseconds (``nvidia-smi`` is the fallback
when the NVML bindings are missing).  Nothing is ever set: clocks, power limits and
other device settings are left as found.  The reference leaves measurement to an
evaluator outside its tree (all2all/task.yml:6-8).
"""
from __future__ import annotations

import statistics
import subprocess
import threading
import time
from typing import Any, Dict, List, Optional

_REASON_BITS = {
    "sw_power_cap": 0x0000000000000004,
    "hw_slowdown": 0x0000000000000008,
    "sw_thermal_slowdown": 0x0000000000000020,
    "hw_thermal_slowdown": 0x0000000000000040,
}


class ClockSampler:
    """``gpu_index`` is the CUDA ordinal; NVML and ``nvidia-smi`` number the physical GPUs and
    ignore ``CUDA_VISIBLE_DEVICES``, so pass the device's ``uuid``
    (``torch.cuda.get_device_properties(i).uuid``) whenever a device mask may be in force:
    the handle is then resolved by UUID and the index is only the fallback."""

    def __init__(self, gpu_index: int, interval_s: float = 0.005, uuid: Optional[str] = None):
        self.gpu_index = gpu_index
        self.uuid = None if not uuid else (uuid if uuid.startswith("GPU-") else "GPU-" + uuid)
        self.interval_s = interval_s
        self._samples: List[tuple] = []  # (sm_mhz, power_w, reasons_mask)
        self._sm_max: Optional[float] = None
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self._nvml = None
        self._handle = None

    def start(self) -> None:
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nvml = pynvml
            self._handle = None
            if self.uuid is not None:
                try:
                    self._handle = pynvml.nvmlDeviceGetHandleByUUID(self.uuid)
                except Exception:  # noqa: BLE001 - older bindings want bytes
                    try:
                        self._handle = pynvml.nvmlDeviceGetHandleByUUID(self.uuid.encode())
                    except Exception:  # noqa: BLE001
                        self._handle = None
            if self._handle is None:
                self._handle = pynvml.nvmlDeviceGetHandleByIndex(self.gpu_index)
            self._sm_max = float(pynvml.nvmlDeviceGetMaxClockInfo(self._handle, pynvml.NVML_CLOCK_SM))
        except Exception:  # noqa: BLE001 - fall back to one nvidia-smi query at stop()
            self._nvml = None
            return
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()

    def _read(self) -> None:
        n = self._nvml
        try:
            sm = float(n.nvmlDeviceGetClockInfo(self._handle, n.NVML_CLOCK_SM))
            power = n.nvmlDeviceGetPowerUsage(self._handle) / 1000.0
            try:
                mask = int(n.nvmlDeviceGetCurrentClocksEventReasons(self._handle))
            except Exception:  # noqa: BLE001
                mask = int(n.nvmlDeviceGetCurrentClocksThrottleReasons(self._handle))
            self._samples.append((sm, power, mask))
        except Exception:  # noqa: BLE001
            pass

    def _run(self) -> None:
        while not self._stop.is_set():
            self._read()
            time.sleep(self.interval_s)

    def stop(self) -> Dict[str, Any]:
        if self._nvml is None:
            return self._smi_once()
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2.0)
        self._read()
        try:
            self._nvml.nvmlShutdown()
        except Exception:  # noqa: BLE001
            pass
        if not self._samples:
            return {"sm_mhz": None, "sm_max_mhz": self._sm_max, "reasons": ["no samples"]}
        pmax = max(p for _, p, _ in self._samples)
        busy = [s for s in self._samples if s[1] >= 0.5 * pmax] or self._samples
        reasons = set()
        for _, _, mask in busy:
            for name, bit in _REASON_BITS.items():
                if mask & bit:
                    reasons.add(name)
        return {
            "sm_mhz": statistics.median(s[0] for s in busy),
            "sm_mhz_min": min(s[0] for s in busy),
            "sm_max_mhz": self._sm_max,
            "power_w_max": pmax,
            "samples": len(self._samples),
            "samples_under_load": len(busy),
            "reasons": sorted(reasons),
        }

    def _smi_once(self) -> Dict[str, Any]:
        fields = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
                  "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
                  "clocks_event_reasons.sw_power_cap")
        try:
            out = subprocess.run(
                ["nvidia-smi", f"--id={self.uuid or self.gpu_index}", f"--query-gpu={fields}", "--format=csv,noheader,nounits"],
                capture_output=True, text=True, timeout=10,
            ).stdout.strip().splitlines()[0]
            parts = [p.strip() for p in out.split(",")]
            names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
            reasons = [n for n, v in zip(names, parts[3:7]) if v.lower().startswith("active")]
            return {"sm_mhz": float(parts[0]), "sm_max_mhz": float(parts[1]), "power_w_max": float(parts[2]),
                    "samples": 1, "reasons": reasons, "note": "single nvidia-smi sample after the timed region"}
        except Exception:  # noqa: BLE001
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["clock query unavailable"]}
