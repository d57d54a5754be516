"""Energy monitor: integrates the GPUs' power draw over a run (read-only NVML / ``nvidia-smi``
queries; no setting of the device is touched).  The reference's SFT loop wires an energy monitor
into its training loop the same way (llama2_sft/primus/src/llama2_custom.py:1295-1893)."""
from __future__ import annotations

import subprocess
import threading
import time


def _read_power_w(indices=None) -> list[float]:
    try:
        import pynvml
        pynvml.nvmlInit()
        n = pynvml.nvmlDeviceGetCount()
        idx = range(n) if indices is None else indices
        return [pynvml.nvmlDeviceGetPowerUsage(pynvml.nvmlDeviceGetHandleByIndex(i)) / 1000.0 for i in idx]
    except Exception:
        pass
    try:
        out = subprocess.run(["nvidia-smi", "--query-gpu=power.draw", "--format=csv,noheader,nounits"], capture_output=True,
                             text=True, timeout=5).stdout
        vals = [float(v) for v in out.split() if v.replace(".", "", 1).isdigit()]
        return vals if indices is None else [vals[i] for i in indices if i < len(vals)]
    except Exception:
        return []


class EnergyMonitor:
    def __init__(self, interval_s: float = 0.5, indices=None, reader=None):
        self.interval, self.indices = interval_s, indices
        self._read = reader or (lambda: _read_power_w(indices))
        self._stop = threading.Event()
        self._thread = None
        self.joules = 0.0
        self.samples = 0
        self.peak_w = 0.0

    def start(self) -> "EnergyMonitor":
        def loop():
            last = time.monotonic()
            while not self._stop.wait(self.interval):
                now = time.monotonic()
                p = sum(self._read())
                self.joules += p * (now - last)
                self.peak_w = max(self.peak_w, p)
                self.samples += 1
                last = now
        self._thread = threading.Thread(target=loop, name="energy-monitor", daemon=True)
        self._thread.start()
        return self

    def stop(self) -> dict:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2 * self.interval + 1)
        return {"energy_j": self.joules, "energy_kwh": self.joules / 3.6e6, "peak_w": self.peak_w, "samples": self.samples}
