"""Host arithmetic of bench.py on CPU: the roofline record of the dominant kernel from a per-launch profile (which
peak it divides by, the event-overhead correction, the traffic figure), and the Zipf token stream."""
import importlib.util
import os

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench():
    spec = importlib.util.spec_from_file_location("bench_under_test", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_roofline_record_from_a_profile():
    b = _bench()
    pk = b.peaks()
    # 100 GEMM launches of 10 us with 4 TFLOP each step, 100 other launches of 5 us; the live step takes 1.0 ms
    prof = {"gemm_bf16:NN:8192x384x384:b1:s1:c0:bn192": {"launches": 60, "ms": 0.6, "flops": 2.4e11, "bytes": 1.0e9},
            "gemm_bf16:NT:8192x384x1152:b1:s1:c0:bn192": {"launches": 40, "ms": 0.4, "flops": 1.6e11, "bytes": 1.0e9},
            "rmsnorm_bwd": {"launches": 100, "ms": 0.5, "flops": 0.0, "bytes": 0.0}}
    r = b.roofline(prof, step_ms=1.0, timed_region_s=0.1, clocks={"reasons": []})
    assert r["bound"] == "tensor" and r["unit"] == "TFLOP/s"
    assert abs(r["achieved"] - 4.0e11 / 1.0e-3 / 1e12) < 1e-9            # 400 TFLOP/s over 1.0 ms of GEMM time
    assert r["peak"] == pk["burst"] and abs(r["frac"] - r["achieved"] / pk["burst"]) < 1e-12
    assert r["launches_per_step"] == 100 and abs(r["ms_per_step"] - 1.0) < 1e-12
    # 1.5 ms of event-bracketed launches for a 1.0 ms step: 2.5 us of overhead per launch, 0.75 ms of GEMM time net
    assert abs(r["event_overhead_us_per_launch"] - 2.5) < 1e-9
    assert abs(r["achieved_net_of_event_overhead"] - 4.0e11 / 0.75e-3 / 1e12) < 1e-6
    assert r["traffic"] == b.GEMM_DRAM_TRAFFIC["bytes_per_step"] / b.GEMM_DRAM_TRAFFIC["launches_per_step"]
    # seconds-long region or a power cap seen: the sustained peak
    assert b.roofline(prof, 1.0, 3.0, {"reasons": []})["peak"] == pk["sustained"]
    assert b.roofline(prof, 1.0, 0.1, {"reasons": ["sw_power_cap"]})["peak"] == pk["sustained"]
    assert b.roofline({"adam": {"launches": 1, "ms": 0.1, "flops": 0.0, "bytes": 0.0}}, 1.0, 0.1, None) is None


def test_zipf_stream_is_seeded_and_in_range():
    b = _bench()
    a = b.zipf_ids(10000, 31769, seed=1)
    assert a.dtype == np.uint32 and a.min() >= 0 and a.max() < 31769
    assert np.array_equal(a, b.zipf_ids(10000, 31769, seed=1))
    assert not np.array_equal(a, b.zipf_ids(10000, 31769, seed=2))
    # rank 1 of a Zipf(1.1) law over 31,769 ranks holds about a tenth of the mass
    assert 0.05 < float((a == 0).mean()) < 0.2
