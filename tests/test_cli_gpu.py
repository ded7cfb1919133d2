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


def test_greedy_generation_equals_the_plain_implementation(tmp_path):
    """-t 0 through the command line, true 32-bit, against the plain implementation on the same
    seeded weights: the same tokens, up to the first stop token (which the command does not print)."""
    import torch
    from plain_qwen3 import PlainQwen3
    from rocml_b200.config import CATALOG, config_from_dict
    from rocml_b200.weights import write_random_model
    entry = CATALOG["tiny-b"]
    folder = str(tmp_path / "tiny_b")
    write_random_model(folder, config_from_dict(entry.config), seed=4)     # what --random --seed-weights 4 writes
    ids = [5, 17, 3, 200, 41]
    want = PlainQwen3(folder, dtype=torch.float32).greedy(ids, 12)
    stops = entry.config.get("eos_token_id", [])
    stops = set(stops if isinstance(stops, list) else [stops])
    cut = next((i for i, t in enumerate(want) if t in stops), len(want))
    p = run("generate", "--model", "tiny-b", "--random", "--seed-weights", "4", "--dtype", "float32",
            "--prompt-ids", ",".join(map(str, ids)), "-n", "12", "-t", "0")
    assert p.returncode == 0, p.stderr[-2000:]
    assert [int(x) for x in p.stdout.split()] == want[:cut]
    assert cut >= 3          # the comparison covers several tokens
    q = run("generate", "--model", folder, "--dtype", "float32", "--prompt-ids", ",".join(map(str, ids)), "-n", "12",
            "-t", "0")       # the same folder by path
    assert q.returncode == 0 and q.stdout == p.stdout


def test_generate_profile_prints_the_table():
    p = run("generate", "--model", "tiny-b", "--random", "--prompt-ids", "5,17,3", "-n", "5", "-t", "0", "--profile")
    assert p.returncode == 0, p.stderr[-2000:]
    assert "== prefill:" in p.stdout and "== decode:" in p.stdout and "what to work on" in p.stdout
    for label in ("q_proj+k_proj+v_proj", "o_proj", "gate_proj+up_proj", "down_proj", "lm_head", "mixer_norm", "embedding"):
        assert label in p.stdout, label


def test_bench_json_keys():
    p = run("bench", "--model", "tiny-a", "--random", "--prompt-tokens", "20", "--decode-tokens", "8", "--runs", "2",
            "--batch", "3", "--json")
    assert p.returncode == 0, p.stderr[-2000:]
    d = json.loads(p.stdout.strip().splitlines()[-1])
    assert d["prompt_tokens"] == 20 and d["decode_tokens"] == 8 and d["runs"] == 2
    assert d["prompt_tokens_per_sec_median"] > 0 and d["decode_tokens_per_sec_median"] > 0
    roof = d["roofline"]
    assert 0 < roof["decode_frac_of_bandwidth"] < 1.2 and 0 < roof["prefill_frac_of_peak_flops"] < 1.2
    assert roof["decode_bytes_per_step"] > 0 and "profile" not in d


def test_bench_profile_json(tmp_path):
    path = str(tmp_path / "profile.json")
    p = run("bench", "--model", "tiny-a", "--random", "--prompt-tokens", "20", "--decode-tokens", "6", "--runs", "1",
            "--batch", "2", "--json", "--profile-json", path)
    assert p.returncode == 0, p.stderr[-2000:]
    d = json.loads(p.stdout.strip().splitlines()[-1])
    with open(path) as f:
        rep = json.load(f)["report"]
    assert [ph["phase"] for ph in rep["phases"]] == ["prefill", "decode"] == [ph["phase"] for ph in d["profile"]["phases"]]
    dec = rep["phases"][1]
    assert dec["steps"] == 5 and dec["tokens"] == 10      # 6 new tokens: the prompts' step samples the first
    assert all(r["elapsed_ms"] > 0 and r["bytes"] > 0 for r in dec["by_op"])


def test_unknown_model_is_an_error_with_the_known_names():
    p = run("generate", "--model", "qwen9-1b")
    assert p.returncode == 1 and "qwen3-8b" in p.stderr
