"""Samples SM clocks and throttle reasons with `nvidia-smi` while a timed region runs, so a
benchmark number can be rejected when the GPU was thermally throttled or clock-locked.
Reading only: no setting of the GPU is ever changed."""
import statistics
import subprocess

_QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
          "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
          "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")


class ClockSampler:
    def __init__(self, gpu_index=0, period_ms=200):
        self._gpu, self._period, self._proc = int(gpu_index), int(period_ms), None

    def __enter__(self):
        try:
            self._proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={_QUERY}", "--format=csv,noheader,nounits", "-i", str(self._gpu),
                 "-lms", str(self._period)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self._proc = None
        return self

    def __exit__(self, *exc):
        self.result = self._finish()
        return False

    def _finish(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "power_w": None, "reasons": [], "samples": 0}
        if self._proc is None:
            return out
        self._proc.terminate()
        try:
            text, _ = self._proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self._proc.kill()
            text, _ = self._proc.communicate()
        clocks, watts, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in text.splitlines():
            cells = [c.strip() for c in line.split(",")]
            if len(cells) < 9:
                continue
            try:
                clocks.append(float(cells[1]))
                out["sm_max_mhz"] = float(cells[2])
            except ValueError:
                continue
            try:
                watts.append(float(cells[3]))
            except ValueError:
                pass
            for name, cell in zip(names, cells[5:9]):
                if cell.lower() == "active":
                    reasons.add(name)
        if clocks:
            out["sm_mhz"] = statistics.median(clocks)
        if watts:
            out["power_w"] = statistics.median(watts)
        out["reasons"], out["samples"] = sorted(reasons), len(clocks)
        return out
