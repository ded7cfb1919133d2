#!/usr/bin/env python3
"""Decode and prefill throughput of the engine at Qwen3-8B layer sizes, random bfloat16 weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--impl reference]
    python bench.py --workload 4b-long | 32b

A step is one decode step of the default batch (8 sequences, prompts of 1,024 tokens, cache
sized for a context of 4,096 per sequence).  One JSON line goes to stdout:

* ``value``: decoded tokens per second, the median of three runs of K steps each, timed on the device
  with CUDA events; the ids sampled by the argmax kernel feed the next step on the device.
* ``e2e``: the same through the Python entry point (``Engine.generate``): every step copies its
  integers (positions, lengths, slots) from pinned host memory and reads the sampled ids back to the
  host; the loop enqueues a step, fed on the device with the ids just sampled, before it reads them.
* ``prefill``: one prompt of 2,048 tokens; ``frac`` = flops / time / measured bf16 peak.
* ``roofline``: bytes a decode step must read (every weight once + the live sequences' cache)
  / time, against the measured copy bandwidth.
* ``points``: decode at batch 1 and 64, and the true 32-bit path (decode at batch 8 and the prompt
  of 2,048 tokens, on ``fp32_layers`` of the layers: it is there to show faults, not to serve).

``--workload`` runs one of the two larger workloads whole through ``Engine.generate`` instead and
prints its own JSON line (see ``rocml_b200.measure.workload``).  Sweeps, timelines and kernel
measurements are ``python -m rocml_b200.measure``.

The engine works on one GPU: for ``--gpus`` above 1 it says so and exits with 2.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FP32_LAYERS = 4


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=int(os.environ.get("WORLD_SIZE", "1")))
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the configuration has (0: all)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--skip-points", action="store_true", help="leave out batch 1 and 64 and the 32-bit path")
    ap.add_argument("--workload", default=None, choices=["4b-long", "32b"],
                    help="instead of the bench line: a whole generation of that workload through Engine.generate")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "xmiksay/rocml is a Rust + HIP (ROCm, gfx1101) workspace with no Python package; "
                          "it needs cargo, hipcc and a GGUF checkpoint, none of which exist here"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine works on one GPU; --gpus {args.gpus} is not supported")
        return 2

    from rocml_b200 import measure as M
    if args.workload:
        print(json.dumps(M.workload(args.workload, args.layers)))
        return 0
    steps, warmup = max(1, args.steps), max(3, args.warmup)

    import torch
    pk = M.peaks()
    max_slots = 64
    cfg, n_full, eng = M.build_engine(args.layers, max_tokens=max_slots * (M.PROMPT + 64 * 5), max_slots=max_slots)
    layers = cfg.num_hidden_layers
    vocab = cfg.vocab_size
    dev_gb = torch.cuda.memory_allocated() / 1e9

    prefill_ms = M.time_prefill(eng, vocab)
    pf = M.prefill_flops(eng, M.PREFILL_TOKENS)

    clocks = M.Clocks()
    clocks.start()
    runs = [M.time_decode(eng, M.BATCH, steps, warmup, vocab, seed=1 + r) for r in range(3)]
    clk = clocks.stop()
    ms, ctx_tokens, launched = sorted(runs)[1]          # the median run of K steps
    value = M.BATCH * 1000.0 / ms
    bytes_step = eng.model.weight_bytes_per_step() + ctx_tokens * eng.kv_bytes_per_token()
    achieved = bytes_step / (ms * 1e-3) / 1e9

    points = {}
    if not args.skip_points:
        for b in (1, 64):
            k = max(16, min(steps, 64))
            m, _, _ = M.time_decode(eng, b, k, warmup, vocab, seed=10 + b)
            points[f"decode_b{b}"] = round(b * 1000.0 / m, 1)

    e2e, h2d, d2h = M.e2e_decode(eng, M.BATCH, min(steps, 128), warmup, vocab)

    if not args.skip_points:
        del eng
        torch.cuda.empty_cache()
        f32 = M.float32_point(FP32_LAYERS)
        points["fp32_decode_b8"] = f32["decode_b8_tok_s"]
        points["fp32_decode_frac_hbm"] = f32["decode_frac_hbm"]
        points["fp32_prefill_2048"] = f32["prefill_tok_s"]
        points["fp32_prefill_tflops"] = f32["prefill_tflops"]

    line = {
        "metric": "decode tok/s at batch 8 (Qwen3-8B layer sizes, bf16, random weights, prompts of 1024)",
        "value": round(value, 1), "unit": "tok/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: seeded uniform-random token ids, random-init weights",
        "config": {
            "model": "Qwen3-8B layer sizes", "layers": layers, "layers_full": n_full,
            "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
            "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": vocab,
            "tied_head": cfg.tie_word_embeddings, "global_batch": M.BATCH, "prompt_len": M.PROMPT,
            "seq_len": M.CTX, "value_is": "median of 3 runs of `steps` decode steps", "parallelism": "single GPU",
            "l2": "inputs larger than L2: every step reads all weights (GB: %.1f)" % (bytes_step / 1e9),
            "device_gb": round(dev_gb, 1), "peaks": pk["source"], "fp32_layers": FP32_LAYERS,
        },
        "clocks": clk,
        "e2e": {"value": round(e2e, 1), "unit": "tok/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": launched,
        "prefill": {"value": round(M.PREFILL_TOKENS * 1000.0 / prefill_ms, 1), "tokens": M.PREFILL_TOKENS,
                    "ms": round(prefill_ms, 3), "frac": round(pf / (prefill_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
