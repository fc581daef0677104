"""CPU: the work accounting bench.py reports rooflines from, against the figures the path's definition gives."""
import importlib.util
import os

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def load_bench():
    spec = importlib.util.spec_from_file_location("bench_module", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_flop_and_byte_counts_of_the_benchmark_shapes():
    b = load_bench()
    cfg = dict(b.CFG_1GPU)
    T, d, E, k, f = cfg["T"], cfg["d"], cfg["E"], cfg["k"], cfg["f"]
    assert (T, d, E, k, f) == (8192, 4096, 64, 8, 1408)
    w = b.algorithmic_work(cfg)
    R = T * k
    gemm = sum(v for bound, v in w.values() if bound == "tensor")
    assert gemm == 18 * R * d * f                       # forward 6 R d f, backward 12 R d f
    assert abs(gemm - 6.80e12) < 0.01e12
    assert w["prepare_experts"] == ("hbm", 2 * T * d + 2 * R * d + 4 * R)
    assert w["merge_experts"] == ("hbm", 2 * R * d + 4 * T * d + 8 * R)
    ep = dict(b.CFG_EP)
    assert ep["T"] == 32768 and 18 * ep["T"] * ep["k"] * ep["d"] * ep["f"] == 27212912787456
    x = b.exchange_work(ep, 8)
    assert x["dispatch"] == 2 * ep["T"] * ep["k"] * ep["d"] * 7 / 8     # 7/8 of the routed rows cross NVLink
    assert b.exchange_work(ep, 2)["dispatch"] == 2 * ep["T"] * ep["k"] * ep["d"] / 2


def test_peaks_come_from_the_measured_file_or_the_stated_fallback():
    b = load_bench()
    p = b.read_peaks()
    assert p["source"] in ("measured", "fallback")
    assert 3000 < p["hbm_gbs"] < 9000 and 800 < p["bf16_tflops_sustained"] <= p["bf16_tflops"] < 2500
