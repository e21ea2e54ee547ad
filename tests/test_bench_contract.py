"""What bench.py owes its caller without a GPU: the line for more than one GPU, the reference arm's line, and that
every size of the timed configuration is named flat in `config` (at most 20 keys, no lists)."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run(*args):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True, timeout=300)


def test_more_than_one_gpu_prints_one_line_and_exits_2():
    r = run("--gpus", "2")
    assert r.returncode == 2
    assert len(r.stdout.strip().splitlines()) == 1 and "one GPU" in r.stdout


def test_reference_arm_says_why_it_is_unavailable():
    r = run("--impl", "reference", "--gpus", "1", "--steps", "4", "--warmup", "3")
    assert r.returncode == 0
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and isinstance(line["unavailable"], str) and "\n" not in line["unavailable"]


def test_the_timed_configurations_are_the_baselines():
    sys.path.insert(0, ROOT)
    import bench
    small, medium, xl = bench.GPT2["small"], bench.GPT2["medium"], bench.GPT2["xl"]
    assert (small["n_layer"], small["n_embd"], small["n_head"], small["n_inner"], small["vocab_size"], small["n_positions"]) == (12, 768, 12, 3072, 50257, 1024)
    assert (medium["n_layer"], medium["n_embd"], medium["n_head"], medium["n_inner"]) == (24, 1024, 16, 4096)
    assert (xl["n_layer"], xl["n_embd"], xl["n_head"], xl["n_inner"]) == (48, 1600, 25, 6400)
    for cfg in (small, medium, xl):
        assert cfg["activation_function"] == "gelu_new" and cfg["layer_norm_epsilon"] == 1e-5
