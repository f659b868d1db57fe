"""Host-side pieces of bench.py that need no GPU: the clock sampler against a fake NVML, the traffic
arithmetic of the roofline object, and the reference arm's JSON line."""
import json
import os
import subprocess
import sys
import time
import types

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import bench  # noqa: E402


class _FakeNvml(types.ModuleType):
    NVML_CLOCK_SM = 1

    def __init__(self, clocks, masks):
        super().__init__("pynvml")
        self.clocks, self.masks, self.calls = list(clocks), list(masks), 0

    def nvmlInit(self):
        pass

    def nvmlDeviceGetHandleByIndex(self, index):
        return ("gpu", index)

    def nvmlDeviceGetHandleByPciBusId(self, bus_id):
        raise RuntimeError("no such device")            # the sampler falls back to the index

    def nvmlDeviceGetMaxClockInfo(self, handle, which):
        return 1965

    def nvmlDeviceGetClockInfo(self, handle, which):
        self.calls += 1
        return self.clocks[min(self.calls, len(self.clocks)) - 1]

    def nvmlDeviceGetCurrentClocksThrottleReasons(self, handle):
        return self.masks[min(self.calls, len(self.masks)) - 1]


def test_clock_sampler_reports_only_samples_inside_the_timed_region(monkeypatch):
    fake = _FakeNvml(clocks=[300] * 3 + [1965] * 10000, masks=[0x8] * 3 + [0x4] * 10000)   # idle and hw_slowdown before the region
    monkeypatch.setitem(sys.modules, "pynvml", fake)
    s = bench.ClockSampler(0)
    time.sleep(0.05)                      # polling before the region: the first samples must not count
    assert fake.calls >= 3
    s.begin()
    time.sleep(0.05)
    s.end()
    time.sleep(0.02)
    out = s.stop()
    assert out["samples"] >= 5 and out["sm_mhz"] == 1965.0 and out["sm_max_mhz"] == 1965.0
    assert out["reasons"] == ["sw_power_cap"]            # the hw_slowdown samples lie before begin()
    assert "NVML" in out["source"]


def test_clock_sampler_decodes_every_rejecting_reason(monkeypatch):
    fake = _FakeNvml(clocks=[1200] * 10000, masks=[0x8 | 0x20 | 0x40] * 10000)
    monkeypatch.setitem(sys.modules, "pynvml", fake)
    s = bench.ClockSampler(0)
    s.begin()
    time.sleep(0.03)
    s.end()
    out = s.stop()
    assert out["reasons"] == ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown"] and out["sm_mhz"] == 1200.0


def test_row_kernel_traffic_follows_the_rows_and_stays_below_the_algorithmic_bytes():
    full = bench.row_kernel_traffic(8192, 32768)
    alg = bench.algorithmic_bytes(8192, 32768)
    assert alg == 4 * 8192 * 32768 * 4 + 8192 * 16
    assert 0.97 * alg < full < alg                       # the L2 residue is the only difference
    half = bench.row_kernel_traffic(4096, 32768)
    assert abs((full - half) - alg / 2) < 1e-3 * alg     # reads and writes grow with the rows, the residue does not


@pytest.mark.timeout(600)
def test_reference_arm_prints_the_contract_line():
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "1", "--rows", "256"],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-1000:]
    line = json.loads([l for l in r.stdout.splitlines() if l.startswith("{")][-1])
    assert line["impl"] == "reference" and line["metric"] == bench.METRIC and line["unit"] == bench.UNIT
    assert line["gpu_launches"] == 0 and line["e2e"]["h2d_bytes_per_step"] == 0 and line["e2e"]["value"] == line["value"]
    assert line["cpu_baseline"]["kind"] in ("port", "reference") and line["cpu_baseline"]["cores"] >= 1
