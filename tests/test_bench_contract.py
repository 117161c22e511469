"""The reference arm of the benchmark runs on host cores only; its JSON line carries the keys
the benchmark contract asks for."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_one_contract_line():
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1",
                          "--warmup", "1", "--sample-rows", "256"], capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["n_gpus"] == 1 and line["higher_is_better"] is True
    assert line["metric"] == "nvfp4_linear_fwd_bwd_tflops" and line["unit"] == "TFLOP/s" and line["value"] > 0
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert line["cpu_baseline"]["value"] == line["value"] == line["e2e"]["value"]
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["e2e"]["d2h_bytes_per_step"] == 0
    assert line["gpu_launches"] == 0 and "workload" in line["config"]
    assert line["steps"] == 1 and line["warmup"] == 1
    # both arms print the same `config` object for the default workload
    sys.path.insert(0, ROOT)
    import bench
    assert line["config"] == bench.base_config(1)


def test_config1_cpu_baseline_runs_and_reports_cores():
    sys.path.insert(0, ROOT)
    import bench
    r = bench.cpu_config1_baseline(reps=3)
    assert r["value"] > 0 and r["cores"] >= 1 and r["runs"] == 3 and "512" in r["workload"]
