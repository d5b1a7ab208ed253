"""The parts of bench.py that run without a GPU: the reference arm (the oracle's torch-CPU
dequantise-then-matmul timed on the host cores) prints one JSON line with the contract's keys,
and the serving key is built from the committed result files."""
import importlib.util
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench_module():
    spec = importlib.util.spec_from_file_location("bench_under_test", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_reference_arm_line_has_the_contract_keys():
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference",
                          "--steps", "1", "--warmup", "3"], capture_output=True, text=True,
                         timeout=600, cwd=ROOT)
    assert res.returncode == 0, res.stderr[-2000:]
    line = json.loads(res.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["higher_is_better"] is True
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "scaling",
                "dtype", "data", "config", "cpu_baseline", "e2e"):
        assert key in line, key
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["e2e"]["d2h_bytes_per_step"] == 0
    assert line["e2e"]["value"] == line["value"] and line["value"] > 0
    assert "workload" in line["config"]


def test_serving_key_reads_the_recorded_result_files():
    serving = _bench_module().recorded_serving()
    assert "recorded" in serving["source"]
    runs = serving["runs"]
    assert runs, "no result files under profiles/serving"
    ours = [r for r in runs if r["kernels"].startswith("this package")]
    stock = [r for r in runs if r["kernels"].startswith("stock")]
    assert ours and stock
    for r in runs:
        assert r["output_throughput"] > 0 and r["total_token_throughput"] >= r["output_throughput"]
        assert os.path.exists(os.path.join(ROOT, r["file"]))
    # same box, same weights, same concurrency: the plug-in column is the faster one
    for s in stock:
        mate = [o for o in ours if o["gpus"] == s["gpus"] and o["concurrency"] == s["concurrency"]]
        assert mate and mate[0]["output_throughput"] > s["output_throughput"]
