"""bench.py's clock sampler picks nvidia-smi's lines by their time stamps: the ones inside the timed region, or - when
the region was shorter than the sampling period - the ones of the warm-up just before it.  No GPU, no nvidia-smi: the
log file is written by the test."""
import datetime
import importlib.util
import os
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def load_bench():
    spec = importlib.util.spec_from_file_location("bench_under_test", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def stamp(t):
    return datetime.datetime.fromtimestamp(t).strftime("%Y/%m/%d %H:%M:%S.%f")[:-3]


def write_log(path, rows):
    with open(path, "w") as f:
        for t, sm, reasons in rows:
            flags = ["Active" if r in reasons else "Not Active" for r in ("hw", "hwt", "swt", "pwr")]
            f.write(f"{stamp(t)}, {sm}, 1965, {', '.join(flags)}\n")


def test_lines_inside_the_timed_region_are_used(tmp_path):
    bench = load_bench()
    s = bench.ClockSampler(0)
    s.path = str(tmp_path / "clocks.csv")
    s.proc = type("P", (), {"terminate": lambda self: None, "wait": lambda self, timeout=None: 0})()
    now = time.time()
    s.t_begin = now - 0.10
    write_log(s.path, [(now - 0.50, 1200, {"pwr"}), (now - 0.08, 1965, set()), (now - 0.05, 1950, set()), (now - 0.02, 1965, set())])
    out = s.stop()
    assert out["samples"] == 3 and out["sm_mhz"] == 1965 and out["reasons"] == [] and out["window"] == "timed region"


def test_a_region_shorter_than_the_sampling_period_falls_back_to_the_warm_up(tmp_path):
    bench = load_bench()
    s = bench.ClockSampler(0)
    s.path = str(tmp_path / "clocks.csv")
    s.proc = type("P", (), {"terminate": lambda self: None, "wait": lambda self, timeout=None: 0})()
    now = time.time()
    s.t_begin = now - 0.005
    write_log(s.path, [(now - 3.0, 900, {"hw"}), (now - 0.10, 1965, {"pwr"}), (now - 0.03, 1965, set())])
    out = s.stop()
    assert out["samples"] == 2 and out["reasons"] == ["sw_power_cap"] and out["window"].startswith("warm-up")
