"""Host-side pieces of the bench scripts that need no GPU."""
import os
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path[:0] = [ROOT, os.path.join(ROOT, "tests", "golden")]

import bench  # noqa: E402
import bench_variants  # noqa: E402
from cases import rope_tables  # noqa: E402


def test_variant_rope_tables_match_the_fixture_generator():
    cos, sin = bench_variants.rope_tables(40, 128, 5e5, "cpu")
    c0, s0 = rope_tables(40, 128, 5e5)
    assert np.array_equal(cos.numpy(), c0) and np.array_equal(sin.numpy(), s0)


def test_clock_sampler_counts_samples_from_the_mark_on():
    s = bench.ClockSampler(0)

    class Done:
        def terminate(self):
            pass

    s.proc = Done()
    s.samples.append((time.perf_counter(), "1200, 1965, Not Active, Not Active, Not Active, Not Active"))
    s.mark()
    s.samples.append((time.perf_counter(), "1965, 1965, Not Active, Not Active, Not Active, Active"))
    s.samples.append((time.perf_counter(), "1950, 1965, Not Active, Not Active, Not Active, Not Active"))
    s.samples.append((time.perf_counter(), "garbage"))
    r = s.stop()
    assert r == {"sm_mhz": 1957.5, "sm_max_mhz": 1965.0, "reasons": ["sw_power_cap"], "samples": 2}


def test_workload_table_holds_the_benchmark_configurations():
    w = bench.WORKLOADS
    assert w["prefill_128k"]["TQ"] == 32768 and w["prefill_128k"]["T"] == 131072
    assert w["prefill_256k_gqa"]["bq"] == 128 and w["prefill_256k_gqa"]["H"] == 64
    assert w["decode_1m"]["T"] == 1 << 20 and w["decode_1m"]["shards"] == 8
    for name, c in w.items():
        assert len(c["chunks"]) == len(c["keep"]) == len(c["strides"]), name
