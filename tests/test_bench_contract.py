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


def test_reference_arm_prints_one_record_and_exits_0():
    """The arm builds the reference's CPU engine and measures it (one layer here, to keep the test short), or
    says in one line why it could not; it never fails the run."""
    p = run("--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "1", "--layers", "1", "--prompt-len", "16",
            "--prefill-tokens", "32")
    assert p.returncode == 0, p.stderr[-1000:]
    rec = json.loads(p.stdout.strip().splitlines()[-1])
    assert rec["impl"] == "reference"
    if "unavailable" in rec:
        assert "\n" not in rec["unavailable"]
    else:
        assert rec["value"] > 0 and rec["unit"] == "tok/s" and rec["prefill"]["tokens"] == 32
        assert rec["config"]["layers"] == 1 and rec["config"]["layers_full"] == 24
        assert len(rec["config"]) <= 20 and all(not isinstance(v, (dict, list)) for v in rec["config"].values())


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
