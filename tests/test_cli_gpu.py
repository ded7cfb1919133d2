"""The command line on a GPU: generate with random weights of a catalog size, and bench --json."""
import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run(*args):
    return subprocess.run([sys.executable, "-m", "rocml_b200", *args], cwd=ROOT, capture_output=True, text=True,
                          timeout=600)


def test_generate_with_random_weights_of_a_catalog_size():
    p = run("generate", "--model", "tiny-b", "--random", "--prompt-ids", "5,17,3", "-n", "7", "--seed", "3")
    assert p.returncode == 0, p.stderr[-2000:]
    toks = [int(x) for x in p.stdout.split()]
    assert 1 <= len(toks) <= 7 and all(0 <= t < 311 for t in toks)
    assert "decode:" in p.stderr and "loaded: 3 layers, hidden=96, vocab=311" in p.stderr
    q = run("generate", "--model", "tiny-b", "--random", "--prompt-ids", "5,17,3", "-n", "7", "--seed", "3")
    assert q.stdout == p.stdout                       # the preset's sampling is seeded
    g = run("generate", "--model", "tiny-b", "--random", "--prompt-ids", "5,17,3", "-n", "7", "-t", "0")
    assert g.returncode == 0 and len(g.stdout.split()) >= 1


def test_bench_json_keys():
    p = run("bench", "--model", "tiny-a", "--random", "--prompt-tokens", "20", "--decode-tokens", "8", "--runs", "2",
            "--batch", "3", "--json")
    assert p.returncode == 0, p.stderr[-2000:]
    d = json.loads(p.stdout.strip().splitlines()[-1])
    assert d["prompt_tokens"] == 20 and d["decode_tokens"] == 8 and d["runs"] == 2
    assert d["prompt_tokens_per_sec_median"] > 0 and d["decode_tokens_per_sec_median"] > 0


def test_unknown_model_is_an_error_with_the_known_names():
    p = run("generate", "--model", "qwen9-1b")
    assert p.returncode == 1 and "qwen3-8b" in p.stderr
