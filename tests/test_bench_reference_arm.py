"""`bench.py --impl reference` on a machine without a GPU: the CPU arm runs the reference's loops
(the checker under oracle/) on a reduced LDA-shaped problem and prints one JSON line with the
keys the benchmark contract names."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_the_contract_line():
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1",
                          "--warmup", "0", "--cpu-seconds", "1", "--scale", "0.02"],
                         capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference"
    assert line["unit"] == "GFLOP/s" and line["higher_is_better"] is True and line["value"] > 0
    assert line["n_gpus"] == 1 and line["steps"] == 1 and line["warmup"] == 0
    assert line["vs_baseline"] is None and line["dtype"] == "f32" and line["data"] == "synthetic"
    assert line["config"]["workload"].startswith("config2+4: LDA-shaped S ")
    assert line["config"]["workload"].endswith("ops A*S, DDS(A,B,S), B*^S")       # the same string in both arms
    cb = line["cpu_baseline"]
    assert cb["kind"] == "port" and cb["cores"] >= 1 and cb["value"] == line["value"] and cb["sample"]
    assert set(cb["ops_gflops"]) == {"dsmult", "dds", "dsmultT"}
    assert line["e2e"] == {"value": line["value"], "unit": "GFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}


def test_the_library_arm_refuses_to_run_without_a_gpu():
    """No CPU fallback: without a CUDA device the library's own arm stops with a message."""
    import torch
    if torch.cuda.is_available():
        import pytest
        pytest.skip("a CUDA device is present")
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--steps", "1", "--warmup", "0"],
                         capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert out.returncode != 0
    assert "no CPU fallback" in out.stderr and out.stdout.strip() == ""
