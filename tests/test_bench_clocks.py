"""CPU: how bench.py turns nvidia-smi lines into the `clocks` record (samples inside the timed region)."""
import datetime
import importlib.util
import os

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
spec = importlib.util.spec_from_file_location("bench_module", os.path.join(ROOT, "bench.py"))
bench = importlib.util.module_from_spec(spec)
spec.loader.exec_module(bench)

T = datetime.datetime(2026, 1, 2, 3, 4, 5)


def line(ms, mhz, power_cap=False, thermal=False):
    ts = (T + datetime.timedelta(milliseconds=ms)).strftime("%Y/%m/%d %H:%M:%S.%f")[:-3]
    flag = lambda b: "Active" if b else "Not Active"
    return "%s, %d, 1965, Not Active, %s, Not Active, %s" % (ts, mhz, flag(thermal), flag(power_cap))


def at(ms):
    return T + datetime.timedelta(milliseconds=ms)


def test_samples_inside_the_timed_region_are_used():
    lines = [line(0, 300), line(20, 1500), line(40, 1900, True), line(60, 1965, True), line(80, 1800), line(100, 400)]
    c = bench.summarise_clock_lines(lines, at(38), at(70))
    assert c == {"sm_mhz": 1900.0, "sm_max_mhz": 1965.0, "samples": 4, "window": "timed region",
                 "reasons": ["sw_power_cap"]}


def test_thermal_reason_is_reported():
    c = bench.summarise_clock_lines([line(10, 1200, thermal=True)], at(0), at(30))
    assert c["reasons"] == ["hw_thermal_slowdown"] and c["samples"] == 1


def test_clock_mismatch_falls_back_to_the_last_lines():
    lines = [line(ms, 300 + ms) for ms in range(0, 200, 20)]
    c = bench.summarise_clock_lines(lines, at(90000), at(90050))          # stamps an hour off: none inside
    assert c["window"].startswith("last samples") and c["samples"] == 3
    assert c["sm_mhz"] == 300 + 160.0


def test_unreadable_lines():
    assert bench.summarise_clock_lines(["garbage"], at(0), at(1))["samples"] == 0
    c = bench.summarise_clock_lines(["?, 1700, 1965, Not Active, Not Active, Not Active, Not Active"], at(0), at(1))
    assert c["samples"] == 1 and c["window"] == "all samples"
