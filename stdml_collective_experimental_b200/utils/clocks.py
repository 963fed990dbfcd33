"""Read-only sampling of SM clocks and throttle reasons while a timed region
runs (NVML through nvidia-ml-py; nothing is ever set)."""
import statistics
import threading
import time

_REASONS = {
    0x0000000000000008: "hw_slowdown",
    0x0000000000000040: "hw_thermal_slowdown",
    0x0000000000000020: "sw_thermal_slowdown",
    0x0000000000000004: "sw_power_cap",
    0x0000000000000080: "hw_power_brake_slowdown",
}


class ClockSampler:
    def __init__(self, device_index=0, period_s=0.002):
        self.device_index = device_index
        self.period_s = period_s
        self.samples = []
        self.stamps = []      # perf_counter() of every sample
        self.window = [None, None]  # the timed region, see mark_begin / mark_end
        self.reasons = set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        self._nvml = None
        self._handle = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nvml = pynvml
            self._handle = pynvml.nvmlDeviceGetHandleByIndex(device_index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._handle, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nvml = None

    def _sample(self):
        n = self._nvml
        if n is None:
            return
        if True:
            try:
                self.samples.append(n.nvmlDeviceGetClockInfo(self._handle, n.NVML_CLOCK_SM))
                self.stamps.append(time.perf_counter())
                mask = n.nvmlDeviceGetCurrentClocksEventReasons(self._handle) if hasattr(
                    n, "nvmlDeviceGetCurrentClocksEventReasons") else \
                    n.nvmlDeviceGetCurrentClocksThrottleReasons(self._handle)
                for bit, name in _REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass

    def _run(self):
        while not self._stop.is_set():
            self._sample()
            time.sleep(self.period_s)

    def start(self):
        if self._nvml is not None:
            self._stop.clear()
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def mark_begin(self):
        """The timed region starts now (the sampler may have been running through
        the warm-up already, so that short regions still see the GPU under load)."""
        self.window[0] = time.perf_counter()

    def mark_end(self):
        self.window[1] = time.perf_counter()

    def stop(self):
        if self._thread is not None:
            self._sample()  # one more while the GPU is still busy or just done
            self._stop.set()
            self._thread.join()
            self._thread = None
        return self.summary()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                    "samples": 0}
        lo, hi = self.window
        inside = [c for c, t in zip(self.samples, self.stamps)
                  if lo is not None and hi is not None and lo <= t <= hi]
        # a region of a few milliseconds holds few samples: then the median is taken
        # over everything since start(), which is warm-up plus region, all under load
        used = inside if len(inside) >= 3 else self.samples
        return {"sm_mhz": statistics.median(used), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples),
                "samples_in_timed_region": len(inside)}
