"""bin/trace_run, driven as a user drives it: a model folder, a trace on standard input, logits in
files.  The same requests are replayed whole, with their last 32 tokens one by one, and in batches of
unequal lengths (one batch after another, so that slots and pages are used again), in 32-bit and in
bfloat16, and every logit row is compared with the plain implementation."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from tiny_models import CONFIGS, prompt, write_model

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TOL = {"float32": 2e-5, "bfloat16": 2.5e-2}


def build_trace(lengths):
    """Steps and, per step, which (request, position) each written row is."""
    steps, rows = [], []

    def add(entries, end):
        steps.append({"step": len(steps), "entries": entries, "end": end})
        rows.append([(e["id"], e["_pos"][w]) for e in entries for w in e["want"]])

    def entry(rid, lo, hi, want_pos):
        pos = list(range(lo, hi))
        return {"id": rid, "_req": rid, "tokens": (lo, hi), "_pos": pos, "want": [p - lo for p in want_pos]}

    # 1. each request alone and whole; logits at every position
    for i, n in enumerate(lengths):
        add([entry(f"w{i}", 0, n, range(n))], [f"w{i}"])
    # 2. the last 32 tokens one by one after the prefix in one step
    for i, n in enumerate(lengths):
        if n <= 32:
            continue
        head = n - 32
        add([entry(f"d{i}", 0, head, [head - 1])], [])
        for t in range(head, n):
            add([entry(f"d{i}", t, t + 1, [t])], [f"d{i}"] if t == n - 1 else [])
    # 3. and 4. batches of unequal lengths, the last 8 tokens of each decoded; shorter requests end
    # earlier; the second batch starts when the first has ended, on the same slots and pages
    for rnd, order in enumerate([list(range(len(lengths))), list(reversed(range(len(lengths))))]):
        ids = {i: f"b{rnd}_{i}" for i in order}
        heads = {i: max(1, lengths[i] - 8) for i in order}
        add([entry(ids[i], 0, heads[i], [heads[i] - 1]) for i in order], [ids[i] for i in order if heads[i] == lengths[i]])
        at = dict(heads)
        live = [i for i in order if at[i] < lengths[i]]
        while live:
            ends = [ids[i] for i in live if at[i] + 1 == lengths[i]]
            add([entry(ids[i], at[i], at[i] + 1, [at[i]]) for i in live], ends)
            for i in live:
                at[i] += 1
            live = [i for i in live if at[i] < lengths[i]]
    return steps, rows


def run_trace(folder, dtype, steps, tokens_by_req, out_dir, max_tokens):
    lines = []
    for s in steps:
        entries = []
        for e in s["entries"]:
            lo, hi = e["tokens"]
            req = int(e["id"].split("_")[-1].lstrip("wdb")) if "_" in e["id"] else int(e["id"][1:])
            entries.append({"id": e["id"], "tokens": tokens_by_req[req][lo:hi], "want": e["want"]})
        lines.append(json.dumps({"step": s["step"], "entries": entries, "end": s["end"]}))
    proc = subprocess.run(
        [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype, "--out", out_dir,
         "--max-tokens", str(max_tokens)],
        input="\n".join(lines) + "\n", capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-3000:]
    done = [l for l in proc.stdout.splitlines() if l.startswith("done ")]
    assert done == [f"done {s['step']}" for s in steps]


@pytest.mark.parametrize("name", ["B", "D"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_in_every_way_of_cutting(name, dtype, tmp_path):
    from plain_qwen3 import PlainQwen3
    cfg = CONFIGS[name]
    folder = write_model(str(tmp_path / "model"), cfg, seed=31, std=0.05)
    plain = PlainQwen3(folder, dtype=torch.float64)
    lengths = [5, 70, 33, 130, 1, 64]
    toks = [prompt(200 + i, n, cfg["vocab_size"]) for i, n in enumerate(lengths)]
    want = [plain.logits(t) for t in toks]
    steps, rows = build_trace(lengths)
    # the most that is live at once: all six requests of a batch, each rounded up to 64
    max_tokens = sum((n + 63) // 64 * 64 for n in lengths)
    out = str(tmp_path / "out")
    run_trace(folder, dtype, steps, toks, out, max_tokens)
    V = cfg["vocab_size"]
    worst = 0.0
    for s, r in zip(steps, rows):
        path = os.path.join(out, f"{s['step']}.f32")
        if not r:
            assert not os.path.exists(path)
            continue
        got = np.fromfile(path, dtype="<f4").reshape(len(r), V)
        for k, (rid, pos) in enumerate(r):
            req = int(rid.split("_")[-1]) if "_" in rid else int(rid[1:])
            w = want[req][pos].numpy()
            err = np.abs(got[k] - w).max() / np.abs(w).max()
            assert err < TOL[dtype], f"{name} {dtype} step {s['step']} request {rid} position {pos}: {err}"
            worst = max(worst, err)
    print(f"{name} {dtype}: worst relative error {worst:.2e} over {sum(len(r) for r in rows)} rows")


def test_trace_run_refuses_more_than_the_cache_holds(tmp_path):
    cfg = CONFIGS["A"]
    folder = write_model(str(tmp_path / "model"), cfg, seed=1)
    line = json.dumps({"step": 0, "entries": [{"id": "a", "tokens": prompt(1, 60, 256), "want": [59]},
                                              {"id": "b", "tokens": prompt(2, 60, 256), "want": [59]}], "end": []})
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype",
                           "float32", "--out", str(tmp_path / "o"), "--max-tokens", "64"],
                          input=line + "\n", capture_output=True, text=True, timeout=300)
    assert proc.returncode != 0 and "CacheFull" in proc.stderr      # two requests of 60 need two pages of 64
    assert "done 0" not in proc.stdout
