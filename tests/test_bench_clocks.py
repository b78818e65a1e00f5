"""The benchmark's own bookkeeping, without a GPU: which clock samples a summary counts."""

import importlib.util
import os

import pytest


@pytest.fixture(scope="module")
def bench():
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "bench.py")
    spec = importlib.util.spec_from_file_location("bench_under_test", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def rows(times, sm="1965", reasons=("Not Active",) * 4):
    return [(t, [sm, "1965", *reasons]) for t in times]


def test_samples_inside_the_timed_regions_are_counted(bench):
    s = bench.ClockSampler()
    s.rows = rows([0.5, 1.5, 2.5, 9.0]) + [(1.6, ["1200", "1965", "Not Active", "Not Active", "Not Active", "Active"])]
    out = s.summary([(1.0, 2.0), (8.5, 9.5)])
    assert out["samples"] == 3 and out["sm_max_mhz"] == 1965.0 and out["reasons"] == ["sw_power_cap"]
    assert out["sm_mhz"] == 1965.0 and "note" not in out          # the median of 1965, 1200, 1965


def test_a_short_run_without_a_sample_inside_falls_back_to_the_nearest_and_says_so(bench):
    s = bench.ClockSampler()
    s.rows = rows([0.8, 5.0])
    out = s.summary([(1.0, 1.02)])
    assert out["samples"] == 1 and out["sm_mhz"] == 1965.0 and "within 0.5 s" in out["note"]
    s.rows = rows([5.0])
    out = s.summary([(1.0, 1.02)])
    assert out["samples"] == 0 and out["sm_mhz"] is None


def test_malformed_lines_are_skipped(bench):
    s = bench.ClockSampler()
    s.rows = [(1.5, ["[N/A]", "1965", "Not Active", "Not Active", "Not Active", "Not Active"]), (1.6, ["1965"])] + rows([1.7])
    assert s.summary([(1.0, 2.0)])["samples"] == 1
