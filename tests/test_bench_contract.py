"""bench.py's command-line contract that needs no GPU."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run(*args):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True, timeout=300)


def test_more_than_one_gpu_is_refused_with_one_line_and_exit_code_2():
    p = run("--gpus", "2", "--steps", "2", "--warmup", "1")
    assert p.returncode == 2
    assert len(p.stdout.strip().splitlines()) == 1 and "one GPU" in p.stdout


def test_reference_arm_reports_unavailable():
    p = run("--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "1")
    assert p.returncode == 0
    rec = json.loads(p.stdout.strip().splitlines()[-1])
    assert rec["impl"] == "reference" and "unavailable" in rec and "\n" not in rec["unavailable"]


def test_config_is_flat_and_names_both_layer_counts():
    sys.path.insert(0, ROOT)
    import bench
    assert bench.CONFIGS["1.5B"] is bench.CONFIG_1P5B and bench.CONFIG_1P5B["num_hidden_layers"] == 24
    assert (bench.CONFIG_3B["num_hidden_layers"], bench.CONFIG_7B["num_hidden_layers"]) == (32, 44)
    # the matrices a step reads: 3.5 G weights at 3B, 7.2 G at 7B (its head is untied)
    assert 6.5e9 < bench.decode_bytes(bench.CONFIG_3B, 0, 0) < 7.5e9
    assert 14e9 < bench.decode_bytes(bench.CONFIG_7B, 0, 0) < 15e9
    nbytes = bench.decode_bytes(bench.CONFIG_1P5B, 8, 512)
    assert 3.3e9 < nbytes < 3.5e9           # 2.69 GB of weights + 8 x (76.5 MB of state to read + 12.6 MB of keys and values)
    assert 5.0e12 < bench.prefill_flops(bench.CONFIG_1P5B, 2048) < 6.0e12
