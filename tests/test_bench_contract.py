"""The measurement programs' contract that needs no GPU: what `bench.py` does for more than one GPU and
for the reference arm, and the options of `rocml_b200.measure`."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run(*args):
    return subprocess.run([sys.executable, *args], cwd=ROOT, capture_output=True, text=True, timeout=300)


def test_more_than_one_gpu_is_one_line_and_exit_code_2():
    p = run("bench.py", "--gpus", "2", "--steps", "4", "--warmup", "3")
    assert p.returncode == 2
    assert len(p.stdout.strip().splitlines()) == 1 and "one GPU" in p.stdout


def test_the_reference_arm_says_why_it_is_unavailable():
    p = run("bench.py", "--impl", "reference", "--gpus", "1", "--steps", "4", "--warmup", "3")
    assert p.returncode == 0
    d = json.loads(p.stdout.strip())
    assert d["impl"] == "reference" and "Rust" in d["unavailable"] and "\n" not in d["unavailable"]


def test_measure_names_its_measurements():
    p = run("-m", "rocml_b200.measure", "--help")
    assert p.returncode == 0
    for word in ("sweep", "timeline", "sampler", "gemm-decode", "gemm-prefill", "workload", "float32", "profile", "host"):
        assert word in p.stdout
    q = run("-m", "rocml_b200.measure", "workload", "7b")
    assert q.returncode != 0 and "4b-long" in q.stderr


def test_the_workloads_are_the_ones_named():
    from rocml_b200.measure import WORKLOADS
    w = WORKLOADS["4b-long"]
    assert (w["model"], w["ctx"], w["prompts"], w["new_tokens"], w["sampling"]) == \
        ("qwen3-4b", 32768, [30000, 8000, 1000, 17], 128, (0.6, 20, 0.95))
    w = WORKLOADS["32b"]
    assert (w["model"], w["ctx"], w["prompts"], w["new_tokens"], w["sampling"]) == \
        ("qwen3-32b", 2048, ("uniform", 64, 64, 1024), None, None)
