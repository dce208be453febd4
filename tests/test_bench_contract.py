"""``bench.py`` on a machine without a GPU: the arithmetic the reported figures rest on, and the reference arm's
line (the CPU restatement of the reference's attention, ``oracle/sdpa_port.py``) with every key of the contract."""
import importlib.util
import json
import pathlib
import subprocess
import sys

import pytest

ROOT = pathlib.Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def bench():
    spec = importlib.util.spec_from_file_location("bench_under_test", ROOT / "bench.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_algorithmic_work_of_the_named_shapes(bench):
    """Unmasked (query, key) pairs, FLOPs (2 forward + 5 backward products) and bytes of the named workloads."""
    assert bench.pairs(1024, 0, 0) == 1024 * 1025 // 2
    assert bench.pairs(4096, 256, 0) == 1_015_936
    # a window with sinks, against the element-wise predicate
    T, w, s = 300, 64, 4
    want = sum(1 for q in range(T) for k in range(q + 1) if k > q - (w - s) or k < s)
    assert bench.pairs(T, w, s) == want
    f, b = bench.flops(*[bench.WORKLOADS["c2"][i] for i in (0, 1, 2, 4, 5, 6)])
    assert abs((f + b) / 1e9 - 180.56) < 0.01 and abs(f / 1e9 - 51.59) < 0.01
    f, b = bench.flops(*[bench.WORKLOADS["c3"][i] for i in (0, 1, 2, 4, 5, 6)])
    assert abs((f + b) / 1e9 - 233.03) < 0.01
    f, b = bench.flops(*[bench.WORKLOADS["c5"][i] for i in (0, 1, 2, 4, 5, 6)])
    assert abs((f + b) / 1e9 - 30_788) < 1
    fb, bb = bench.algorithmic_bytes(32, 1024, 12, 12, 64)
    assert abs(fb / 1e6 - 202.9) < 0.1 and abs((fb + bb) / 1e6 - 611.8) < 0.1
    fb, bb = bench.algorithmic_bytes(16, 4096, 16, 16, 64)
    assert abs((fb + bb) / 1e6 - 1631.6) < 0.1


def test_reference_arm_prints_the_contract_line():
    r = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0"],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["unit"] == "TFLOP/s" and line["higher_is_better"] is True
    assert line["metric"] == "attention fwd+bwd TFLOP/s (bf16 causal)"
    assert "B=32 H=12 T=1024 D=64" in line["config"]["workload"]
    assert line["value"] > 0 and line["gpu_launches"] == 0
    cpu = line["cpu_baseline"]
    assert cpu["kind"] == "port" and cpu["cores"] >= 1 and cpu["value"] == line["value"] and "batch elements" in cpu["sample"]
    assert line["e2e"] == {"value": line["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
