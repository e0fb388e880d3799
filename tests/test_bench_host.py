"""Host-side pieces of bench.py that need no GPU: the clock sampler's windowing."""
import importlib.util
import os

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
spec = importlib.util.spec_from_file_location("bench_under_test", os.path.join(ROOT, "bench.py"))
bench = importlib.util.module_from_spec(spec)
spec.loader.exec_module(bench)


class _FakeProc:
    def terminate(self):
        pass

    def wait(self, timeout=None):
        return 0


def _row(sm, power_cap="Not Active"):
    return ["0", str(sm), "1965", "500.0", "0x0", "Not Active", "Not Active", "Not Active", power_cap]


def _sampler(rows):
    s = bench.ClockSampler(0)
    s.proc = _FakeProc()
    s.rows = list(rows)
    return s


def test_clock_sampler_uses_the_timed_window():
    s = _sampler([_row(1000), _row(1000), _row(1965), _row(1950), _row(1965), _row(1200)])
    out = s.stop(2, 5)
    assert out["samples"] == 3 and out["sm_mhz"] == 1965.0 and out["sm_max_mhz"] == 1965.0
    assert out["window"] == "timed region" and out["reasons"] == []


def test_clock_sampler_falls_back_to_all_samples_and_reports_reasons():
    s = _sampler([_row(1900), _row(1800, "Active")])
    out = s.stop(2, 2)                      # nothing arrived inside the window
    assert out["samples"] == 2 and out["window"] == "warm-up and timed region"
    assert out["reasons"] == ["sw_power_cap"]


def test_clock_sampler_without_nvidia_smi():
    s = bench.ClockSampler(0)
    assert s.stop()["reasons"] == ["nvidia-smi unavailable"]
