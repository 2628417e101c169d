"""SM clock, power and throttle reasons during a timed region, read through NVML (read-only).
The reference logs the same beside its A/B numbers (backend/node/ab.py:136-157)."""
import threading
import time


class ClockSampler:
    """SM clock, power and throttle reasons of one GPU, read through NVML every 10 ms on a host
    thread; only samples taken while `timed` is set count (the timed region).  Read-only."""
    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, index):
        self.index, self.samples, self.timed, self._stop, self.thread, self.h, self.nv = index, [], False, False, None, None, None

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv, self.h = pynvml, pynvml.nvmlDeviceGetHandleByIndex(self.index)
        except Exception:
            return
        self.thread = threading.Thread(target=self._run, daemon=True)
        self.thread.start()

    def _run(self):
        nv, h = self.nv, self.h
        while not self._stop:
            try:
                if self.timed:
                    try:
                        mask = nv.nvmlDeviceGetCurrentClocksEventReasons(h)
                    except Exception:
                        mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(h)
                    self.samples.append((nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM), nv.nvmlDeviceGetPowerUsage(h) / 1000.0, mask))
            except Exception:
                pass
            time.sleep(0.01)

    def stop(self):
        self._stop = True
        if self.thread is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvml unavailable"]}
        self.thread.join(timeout=1)
        try:
            mx = self.nv.nvmlDeviceGetMaxClockInfo(self.h, self.nv.NVML_CLOCK_SM)
        except Exception:
            mx = None
        sm = sorted(x[0] for x in self.samples)
        reasons = sorted({name for _, _, mask in self.samples for bit, name in self.REASONS.items() if mask & bit})
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "reasons": reasons,
                "power_w_max": max((x[1] for x in self.samples), default=None), "samples": len(sm)}
