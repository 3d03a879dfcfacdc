"""Host logic of the benchmark's measurement loop (no GPU): the visiting order the reference uses
(qual/src/device_benchmark.rs:1228-1239) and how many graph launches make one sample."""
import importlib.util
import os

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench():
    spec = importlib.util.spec_from_file_location("bench_under_test", os.path.join(ROOT, "bench.py"))
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


def test_measurement_order_rotates_and_reverses():
    order = _bench().Protocol.order
    assert order(0, 4) == [0, 1, 2, 3]
    assert order(1, 4) == [2, 1, 0, 3]          # reversed, then rotated by one
    assert order(2, 4) == [2, 3, 0, 1]
    for sample in range(12):
        assert sorted(order(sample, 5)) == [0, 1, 2, 3, 4]   # every case once per sample


def test_operations_per_sample_reach_the_floor():
    bench = _bench()
    proto = bench.Protocol(torch=None)
    floor = bench.Protocol.OPS_PER_SAMPLE
    for ops in (1, 3, 4, 7, 10, 32, 33, 762):
        proto.add(f"case{ops}", lambda: None, ops)
    for name, _replay, ops, inner in proto.cases:
        assert ops * inner >= floor, name
        assert ops * (inner - 1) < floor, name       # no more graph launches than needed
    proto.add("explicit", lambda: None, 4, inner=1)
    assert proto.cases[-1][3] == 1
