"""Thermal telemetry against a stand-in NVML: ring, window summaries, verdicts.  Nothing here touches a GPU."""
import time

from cuteafd_b200.utils import thermal
from cuteafd_b200.utils.thermal import NvmlBackend, Sample, SmiBackend, ThermalMonitor, summarize


class FakeNvml:
    NVML_CLOCK_SM, NVML_CLOCK_MEM, NVML_TEMPERATURE_GPU = 1, 2, 0

    def __init__(self, gpus=2):
        self.n = gpus
        self.state = {g: {"sm": 1965, "mem": 3996, "mw": 400_000, "temp": 55, "reasons": 0} for g in range(gpus)}
        self.inits = self.shutdowns = 0
        self.fail = set()

    def nvmlInit(self): self.inits += 1
    def nvmlShutdown(self): self.shutdowns += 1
    def nvmlDeviceGetCount(self): return self.n
    def nvmlDeviceGetHandleByIndex(self, i): return i

    def nvmlDeviceGetClockInfo(self, h, kind):
        if h in self.fail:
            raise RuntimeError("NVML_ERROR_GPU_IS_LOST")
        return self.state[h]["sm" if kind == self.NVML_CLOCK_SM else "mem"]

    def nvmlDeviceGetMaxClockInfo(self, h, kind): return 1965
    def nvmlDeviceGetPowerUsage(self, h): return self.state[h]["mw"]
    def nvmlDeviceGetTemperature(self, h, kind): return self.state[h]["temp"]
    def nvmlDeviceGetCurrentClocksThrottleReasons(self, h): return self.state[h]["reasons"]


def test_ring_and_windows():
    nv = FakeNvml()
    mon = ThermalMonitor(NvmlBackend(nv), capacity=8)
    t0 = time.monotonic()
    for _ in range(3):
        assert mon.poll() == 2
    nv.state[0].update(sm=1300, mw=1_000_000, reasons=0x4)          # power cap on gpu 0
    t1 = time.monotonic()
    for _ in range(3):
        mon.poll()
    t2 = time.monotonic()
    first, second = mon.window(t0, t1), mon.window(t1, t2)
    assert first[0]["verdict"] == "ok" and first[0]["sm_mhz"]["median"] == 1965 and first[0]["samples"] == 3
    assert second[0]["verdict"] == "power_cap" and second[0]["reasons"] == {"sw_power_cap": 1.0}
    assert second[0]["power_w"]["max"] == 1000.0 and second[1]["verdict"] == "ok"
    assert mon.window(t0, t2, gpu=0)["reasons"]["sw_power_cap"] == 0.5
    # the ring is bounded
    for _ in range(20):
        mon.poll()
    assert len(mon.ring[0]) == 8
    assert mon.latest()[0]["reason_names"] == ["sw_power_cap"]
    # a GPU whose query fails drops out of the reading; the others go on
    nv.fail.add(1)
    assert mon.poll() == 1
    mon.stop()
    assert nv.shutdowns == 1


def test_verdicts():
    def mk(sm, reasons, n=5):
        return [Sample(float(i), 0, sm, 1965.0, 3996.0, 500.0, 60.0, reasons) for i in range(n)]
    assert summarize(mk(1900, 0))["verdict"] == "ok"
    assert summarize(mk(1200, 0x4))["verdict"] == "power_cap"
    assert summarize(mk(1200, 0x40))["verdict"] == "thermal"
    assert summarize(mk(1200, 0x20 | 0x4))["verdict"] == "thermal"
    assert summarize(mk(1000, 0))["verdict"] == "locked"            # slow with no reason: a leftover clock lock
    assert summarize(mk(300, 0x1))["verdict"] == "ok"               # idle clocks are not a lock
    assert summarize([])["verdict"] == "unmeasured"


def test_smi_backend_parses_rows():
    text = ("0, 1965, 1965, 3996, 412.5, 51, Not Active, Not Active, Not Active, Not Active\n"
            "1, 1305, 1965, 3996, 998.1, 74, Active, Not Active, Not Active, Not Active\n"
            "garbage line\n")
    got = SmiBackend(exe="nvidia-smi", run=lambda: text).read()
    assert [s.gpu for s in got] == [0, 1] and got[1].reason_names() == ["sw_power_cap"] and got[0].reasons == 0
    assert got[1].power_w == 998.1 and got[1].temp_c == 74.0


def test_background_thread_samples():
    nv = FakeNvml(1)
    mon = ThermalMonitor(NvmlBackend(nv), period_s=0.01).start()
    time.sleep(0.15)
    mon.stop()
    assert len(mon.ring[0]) >= 3
    rep = mon.report(5.0)
    assert rep["available"] and rep["window"][0]["samples"] >= 3


def test_no_gpu_host_reports_unavailable(monkeypatch):
    monkeypatch.setattr(thermal, "open_backend", lambda gpus=None: None)
    assert thermal.sample_once() == {"available": False}
    assert ThermalMonitor(None).start().report()["available"] is False
