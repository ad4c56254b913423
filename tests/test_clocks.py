"""The clock sampler against a stand-in NVML: it only reads, reports the median SM clock, the
maximum, the peak power and every throttle reason that was active in any sample, and keeps
working when a query is missing."""
import sys
import time
import types

from aboleth_b200.utils.clocks import ClockSampler


def _fake_nvml(clocks, reasons, *, has_event_reasons=True, power=True):
    nv = types.ModuleType("pynvml")
    nv.NVML_CLOCK_SM = 1
    nv.nvmlClocksEventReasonSwPowerCap = 0x4
    nv.nvmlClocksEventReasonHwSlowdown = 0x8
    nv.nvmlClocksEventReasonSwThermalSlowdown = 0x20
    nv.nvmlClocksEventReasonHwThermalSlowdown = 0x40
    nv.nvmlClocksEventReasonHwPowerBrakeSlowdown = 0x80
    state = {"i": 0, "calls": []}

    def record(name):
        state["calls"].append(name)

    nv.nvmlInit = lambda: record("init")
    nv.nvmlDeviceGetHandleByIndex = lambda index: ("gpu", index)
    nv.nvmlDeviceGetMaxClockInfo = lambda handle, kind: 1965

    def clock(handle, kind):
        record("clock")
        value = clocks[min(state["i"], len(clocks) - 1)]
        return value

    def mask(handle):
        record("reasons")
        value = reasons[min(state["i"], len(reasons) - 1)]
        state["i"] += 1
        return value

    nv.nvmlDeviceGetClockInfo = clock
    if power:
        nv.nvmlDeviceGetPowerUsage = lambda handle: 300_000 + 1000 * state["i"]
    if has_event_reasons:
        nv.nvmlDeviceGetCurrentClocksEventReasons = mask
    else:
        nv.nvmlDeviceGetCurrentClocksThrottleReasons = mask
    nv.state = state
    return nv


def _run(nv, samples):
    previous = sys.modules.get("pynvml")
    sys.modules["pynvml"] = nv
    try:
        sampler = ClockSampler(3, period=0.005)
        sampler.start()
        deadline = time.time() + 5
        while nv.state["i"] < samples and time.time() < deadline:
            time.sleep(0.005)
        return sampler.stop()
    finally:
        if previous is None:
            del sys.modules["pynvml"]
        else:
            sys.modules["pynvml"] = previous


def test_median_clock_and_every_reason_seen():
    nv = _fake_nvml([1965, 1965, 1300, 1965, 1965], [0, 0x4, 0x4 | 0x40, 0, 0])
    result = _run(nv, 5)
    assert result["sm_max_mhz"] == 1965 and result["sm_mhz"] == 1965 and result["samples"] >= 5
    assert result["reasons"] == ["hw_thermal_slowdown", "sw_power_cap"]
    assert result["power_w_max"] >= 300.0
    # nothing but queries was called: the sampler never sets anything
    assert set(nv.state["calls"]) <= {"init", "clock", "reasons"}


def test_older_binding_without_event_reasons_and_without_power():
    nv = _fake_nvml([1200, 1200, 1200], [0x8, 0x8, 0x8], has_event_reasons=False, power=False)
    result = _run(nv, 3)
    assert result["sm_mhz"] == 1200 and result["reasons"] == ["hw_slowdown"] and result["power_w_max"] is None


def test_without_nvml_the_record_is_empty_not_an_error():
    broken = types.ModuleType("pynvml")
    broken.nvmlInit = lambda: (_ for _ in ()).throw(RuntimeError("no driver"))
    previous = sys.modules.get("pynvml")
    sys.modules["pynvml"] = broken
    try:
        sampler = ClockSampler(0)
        sampler.start()
        result = sampler.stop()
    finally:
        if previous is None:
            del sys.modules["pynvml"]
        else:
            sys.modules["pynvml"] = previous
    assert result == {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0, "power_w_max": None}
