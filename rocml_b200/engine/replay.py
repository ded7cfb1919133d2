"""Trace replay: feed given token ids through the engine step by step and write logits.

It samples nothing and owns no model code: it parses steps, keeps a map from request ids to
cache slots, calls ``Engine.step`` and writes what comes back.  Steps arrive one JSON object
per line::

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

For a step in which something is wanted, ``<out>/<step>.f32`` receives the logits at the
wanted places, in the order of the entries and of ``want``, as little-endian float32
[wanted, vocab].  After every step ``done <step>`` is printed and flushed.  (The reference's
nearest relatives are its teacher-forced loop, rocml-cli/src/eval/ppl.rs:17-41, and its
serial-versus-chunked harness, rocml/tests/dense_chunked_prefill_parity.rs:128-174.)
"""
from __future__ import annotations

import json
import os
import sys
from typing import Dict, IO

import numpy as np

from ..errors import RocmlError
from .engine import Engine, StepEntry


def replay(engine: Engine, lines: IO[str], out_dir: str, done: IO[str] = sys.stdout) -> int:
    os.makedirs(out_dir, exist_ok=True)
    slots: Dict[str, int] = {}
    n_steps = 0
    for line in lines:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries = []
        for e in rec.get("entries", []):
            rid = str(e["id"])
            if rid not in slots:
                slots[rid] = engine.new_sequence()
            entries.append(StepEntry(slots[rid], e["tokens"], e.get("want", [])))
        logits = engine.step(entries) if entries else None
        if logits is not None:
            arr = logits.detach().to("cpu").numpy().astype("<f4", copy=False)
            tmp = os.path.join(out_dir, f".{step}.f32.tmp")
            arr.tofile(tmp)
            os.replace(tmp, os.path.join(out_dir, f"{step}.f32"))
        for rid in rec.get("end", []):
            rid = str(rid)
            if rid not in slots:
                raise RocmlError(f"step {step} ends request {rid!r}, which never started")
            engine.release(slots.pop(rid))
        n_steps += 1
        print(f"done {step}", file=done, flush=True)
    return n_steps


def main(argv=None) -> int:
    import argparse

    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder that receives <step>.f32")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at once (each rounded up to 64); sizes the cache")
    args = ap.parse_args(argv)
    engine = Engine.from_folder(args.model, dtype=args.dtype, device="cuda:0", max_tokens=args.max_tokens)
    replay(engine, sys.stdin, args.out)
    return 0
