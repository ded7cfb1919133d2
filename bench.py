#!/usr/bin/env python3
"""Decode and prefill throughput of the engine at Qwen3-8B layer sizes, random bfloat16 weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--impl reference]

A step is one decode step of the default batch (8 sequences, prompts of 1,024 tokens, cache
sized for a context of 4,096 per sequence).  One JSON line goes to stdout:

* ``value``: decoded tokens per second over K steps, timed on the device with CUDA events;
  the ids sampled by the argmax kernel feed the next step on the device.
* ``e2e``: the same through the Python entry point (``Engine.generate``): every step copies its
  integers (positions, lengths, slots) from pinned host memory and reads the sampled ids back to the
  host; the loop enqueues a step, fed on the device with the ids just sampled, before it reads them.
* ``prefill``: one prompt of 2,048 tokens; ``frac`` = flops / time / measured bf16 peak.
* ``roofline``: bytes a decode step must read (every weight once + the live sequences' cache)
  / time, against the measured copy bandwidth.
* ``points``: decode at batch 1 and 64.

The engine works on one GPU: for ``--gpus`` above 1 it says so and exits with 2.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

MODEL = "qwen3-8b"          # catalog entry with the benchmark's layer sizes
PROMPT = 1024
PREFILL_TOKENS = 2048
CTX = 4096
BATCH = 8


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


class Clocks:
    """Samples nvidia-smi while a timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.proc, self.path = None, None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        try:
            for line in open(self.path):
                f = [x.strip() for x in line.split(",")]
                if len(f) < 7:
                    continue
                try:
                    sm.append(float(f[0])); smax.append(float(f[1]))
                except ValueError:
                    continue
                for name, v in zip(names, f[3:7]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
            os.remove(self.path)
        except OSError:
            pass
        if sm:
            out = {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(smax), "reasons": sorted(reasons),
                   "samples": len(sm)}
        return out


def build_engine(layers, max_tokens, max_slots):
    import torch
    from rocml_b200.config import CATALOG, config_from_dict
    from rocml_b200.engine import Engine, Model
    from rocml_b200.parts import BuildEnv

    full = dict(CATALOG[MODEL].config)
    n_full = full["num_hidden_layers"]
    if layers:
        full["num_hidden_layers"] = layers
    cfg = config_from_dict(full)
    dev = torch.device("cuda:0")
    with torch.cuda.device(dev):
        model = Model(cfg.to_model_spec(), BuildEnv(dev, torch.bfloat16))
        model.load_random(seed=0)
        eng = Engine(model, max_tokens=max_tokens, max_slots=max_slots, max_step_tokens=4096, max_seq_len=CTX)
    return cfg, n_full, eng


def prompts(n, length, vocab, seed):
    import torch
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n, length), generator=g).tolist()


def time_decode(eng, batch, steps, warmup, vocab, seed):
    """K decode steps of `batch` sequences after prompts of PROMPT tokens, timed with CUDA events.
    Returns (ms per step, mean cache tokens read per step, kernels launched in the timed region)."""
    import torch
    from rocml_b200 import StepEntry, kernels
    slots = [eng.new_sequence() for _ in range(batch)]
    ps = prompts(batch, PROMPT, vocab, seed)
    tok = torch.zeros(max(batch, 1), dtype=torch.int32, device=eng.device)
    logits = eng.step([StepEntry(s, p, [PROMPT - 1]) for s, p in zip(slots, ps)])
    kernels.argmax(logits, tok, batch)

    def one():
        lg = eng.step([StepEntry(s, [0], [0]) for s in slots], device_tokens=tok)
        kernels.argmax(lg, tok, batch)

    for _ in range(warmup):
        one()
    torch.cuda.synchronize()
    k0 = kernels.launch_count + eng.graph_kernel_launches
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ctx_tokens = 0
    start.record()
    for _ in range(steps):
        ctx_tokens += sum(eng.length(s) + 1 for s in slots)
        one()
    end.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(end) / steps
    launched = kernels.launch_count + eng.graph_kernel_launches - k0
    kernels.check_status(eng.device)
    for s in slots:
        eng.release(s)
    return ms, ctx_tokens / steps, launched


def time_prefill(eng, vocab, runs=3, warmup=2):
    import torch
    from rocml_b200 import StepEntry, kernels
    p = prompts(1, PREFILL_TOKENS, vocab, 99)[0]
    times = []
    for i in range(warmup + runs):
        slot = eng.new_sequence()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        eng.step([StepEntry(slot, p, [PREFILL_TOKENS - 1])])
        b.record()
        torch.cuda.synchronize()
        if i >= warmup:
            times.append(a.elapsed_time(b))
        eng.release(slot)
    kernels.check_status(eng.device)
    return statistics.median(times)


def prefill_flops(cfg, layers, T):
    H, I, V = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
    per_layer = H * (cfg.q_dim + 2 * cfg.kv_dim) + cfg.q_dim * H + 3 * H * I
    linear = 2.0 * T * per_layer * layers + 2.0 * V * H           # the head runs on one row
    attn = 4.0 * cfg.num_attention_heads * cfg.head_dim * (T * (T + 1) / 2) * layers   # causal QK^T and PV
    return linear + attn


def e2e_decode(eng, batch, steps, warmup, vocab):
    """Decoded tokens per second through Engine.generate: host token ids in, host token ids out,
    a pinned-memory copy each way in every step."""
    from rocml_b200 import GenerateStats
    ps = prompts(batch, PROMPT, vocab, 7)
    eng.generate(ps, max_new_tokens=max(warmup, 2), stop_tokens=[], ignore_eos=True, max_batch=batch)
    stats = GenerateStats()
    eng.generate(ps, max_new_tokens=steps + 1, stop_tokens=[], ignore_eos=True, max_batch=batch, stats=stats)
    return stats.decode_tokens / stats.decode_seconds, eng.last_h2d_bytes, batch * 4


def micro(which):
    """Kernel microbenchmarks: each kernel launched back to back inside a CUDA graph (no host
    time), at the Qwen3-8B layer sizes.  Results are printed, one line per case; they feed the
    notes under profiles/ and are not part of the bench line."""
    import torch
    from rocml_b200 import kernels
    from rocml_b200.config import CATALOG, config_from_dict
    cfg = config_from_dict(CATALOG[MODEL].config)
    dev = "cuda:0"
    H, I, V = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
    nq, nkv, hd = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim

    def in_graph(fn, reps):
        fn()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(reps):
                fn()
        g.replay()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(); g.replay(); g.replay(); b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) * 1000 / (2 * reps)

    shapes = [("qkv", cfg.q_dim + 2 * cfg.kv_dim, H), ("o", H, cfg.q_dim), ("gate_up", 2 * I, H), ("down", H, I),
              ("head", V, H)]
    if which == "gemm-decode":
        # weights rotate through more than the L2 holds, so every launch streams from HBM
        for M in (1, 8, 64):
            for name, N, K in shapes:
                copies = max(2, int(300e6 / (N * K * 2)) + 1)
                ws = [torch.randn(N, K, device=dev).bfloat16() for _ in range(copies)]
                x = torch.randn(M, K, device=dev).bfloat16()
                for S in (1, 2, 4, 8):
                    if K // 64 < 5 * S or (name == "head" and S > 2):
                        continue
                    out = torch.empty((S, M, N), dtype=torch.float32, device=dev)
                    for stages in (3, 5):
                        it = iter(range(10 ** 9))
                        us = in_graph(lambda: kernels.gemm_tcgen05(x, ws[next(it) % copies], out, None, M, stages), 4 * copies)
                        print(f"gemm decode M={M} {name} N={N} K={K} splits={S} stages={stages}: {us:.1f} us "
                              f"{N * K * 2 / us / 1e6:.2f} TB/s", flush=True)
                del ws
    elif which == "gemm-prefill":
        for name, N, K in shapes[:4]:
            w = torch.randn(N, K, device=dev).bfloat16()
            x = torch.randn(PREFILL_TOKENS, K, device=dev).bfloat16()
            for od in (torch.bfloat16, torch.float32):
                out = torch.empty((PREFILL_TOKENS, N), dtype=od, device=dev)
                us = in_graph(lambda: kernels.gemm_tcgen05(x, w, out, None, PREFILL_TOKENS), 10)
                print(f"gemm prefill M={PREFILL_TOKENS} {name} N={N} K={K} out={str(od)[6:]}: {us:.1f} us "
                      f"{2 * PREFILL_TOKENS * N * K / us / 1e6:.0f} TFLOP/s", flush=True)
        x = torch.randn(PREFILL_TOKENS, H, device=dev).bfloat16()
        w = torch.randn(cfg.q_dim + 2 * cfg.kv_dim, H, device=dev).bfloat16()
        us = in_graph(lambda: torch.matmul(x, w.t()), 10)
        print(f"library matmul (for scale) qkv: {us:.1f} us {2 * PREFILL_TOKENS * w.shape[0] * H / us / 1e6:.0f} TFLOP/s")
    else:
        raise SystemExit(f"unknown --micro {which!r}: gemm-decode, gemm-prefill or timeline")


def sampler_times():
    """Time of one sampling step (kernel, copy of the ids to the host, the host's own part) over logits of the
    benchmark's vocabulary, for the ways of sampling and a few batch sizes; beside it the kernel's own time,
    launched back to back."""
    import torch
    from rocml_b200.config import CATALOG, config_from_dict
    from rocml_b200.sampling import Sampler, SamplingParams
    from rocml_b200.sampling.params import XorShift64Star
    vocab = config_from_dict(CATALOG[MODEL].config).vocab_size
    dev = "cuda:0"
    ways = [("greedy", SamplingParams()), ("temperature 0.6, top-k 20, top-p 0.95", SamplingParams(0.6, top_k=20, top_p=0.95)),
            ("temperature 0.8", SamplingParams(0.8)), ("temperature 0.8, top-p 0.9", SamplingParams(0.8, top_p=0.9)),
            ("temperature 0.8, top-k 2000", SamplingParams(0.8, top_k=2000))]
    for batch in (1, 8, 64):
        logits = torch.randn(batch, vocab, device=dev) * 2.0
        s = Sampler(dev, max_batch=64)
        for name, sp in ways:
            rngs = [XorShift64Star(i) for i in range(batch)]
            for _ in range(3):
                s.sample(logits, [sp] * batch, rngs, [[]] * batch)
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            for _ in range(20):
                s.sample(logits, [sp] * batch, rngs, [[]] * batch)
            wall = (time.perf_counter() - t0) / 20 * 1e6
            # the kernel alone, on the rows that the last step left on the device
            from rocml_b200 import kernels
            run = (lambda: kernels.argmax(logits, s._out, batch)) if sp.is_greedy else \
                (lambda: kernels.sample(logits, batch, s._rows, s._hist, s._out))
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(20):
                run()
            b.record()
            torch.cuda.synchronize()
            print(f"batch {batch:3d}  {name:40s} {wall:8.1f} us a step, kernel {a.elapsed_time(b) / 20 * 1e3:7.1f} us")


def sweep(cases=None, steps=32):
    """Decode steps at other batch sizes and context lengths than the bench line's: milliseconds a step,
    tokens a second, and the bytes a step has to read (weights once, the live cache) over its time, as a
    fraction of the measured copy bandwidth.  All layers of the configuration; prompts are fed in pieces
    of at most 4,096 tokens."""
    import torch
    from rocml_b200 import StepEntry, kernels
    global CTX
    cases = cases or [(1, 1024), (1, 8192), (1, 32000), (4, 16000), (8, 1024), (8, 8192), (8, 32000), (16, 2048),
                      (32, 1024), (32, 8192), (64, 1024), (64, 4000), (128, 1024), (256, 1024)]
    pk = peaks()
    print("batch  context  ms/step    tok/s   GB/step   GB/s  of %s copy bandwidth" % pk["source"])
    for batch, ctx in cases:
        CTX = ctx + 256
        cfg, n_full, eng = build_engine(0, batch * ((ctx + 256 + 63) // 64 * 64), batch)
        slots = [eng.new_sequence() for _ in range(batch)]
        ps = prompts(batch, ctx, cfg.vocab_size, 3)
        tok = torch.zeros(batch, dtype=torch.int32, device=eng.device)
        piece = max(64, (4096 // batch) // 64 * 64)
        for lo in range(0, ctx, piece):
            hi = min(ctx, lo + piece)
            logits = eng.step([StepEntry(s, p[lo:hi], [hi - lo - 1]) for s, p in zip(slots, ps)])
        kernels.argmax(logits, tok, batch)

        def one():
            kernels.argmax(eng.step([StepEntry(s, [0], [0]) for s in slots], device_tokens=tok), tok, batch)

        for _ in range(6):
            one()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(steps):
            one()
        b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b) / steps
        gb = (eng.model.weight_bytes_per_step() + batch * (ctx + 6 + steps / 2) * eng.kv_bytes_per_token()) / 1e9
        print(f"{batch:5d} {ctx:8d} {ms:8.3f} {batch / ms * 1e3:8.0f} {gb:9.2f} {gb / ms * 1e3:6.0f}  {gb / ms * 1e3 / pk['hbm_gbs']:.2f}",
              flush=True)
        kernels.check_status(eng.device)
        del eng, slots, logits
        torch.cuda.empty_cache()


def timeline(batch=BATCH, layers=4):
    """Where a decode step's time goes, kernel by kernel, as the step really runs (inside its CUDA
    graph, kernels overlapping their predecessors through programmatic dependent launch): start and
    end of every kernel from the profiler's activity records (CUPTI, no kernel is replayed), and for
    each kernel the time from its predecessor's end to its own end, which is what it adds to the step."""
    import torch
    from torch.profiler import ProfilerActivity, profile
    from rocml_b200 import StepEntry, kernels
    cfg, n_full, eng = build_engine(layers, batch * (PROMPT + 256), batch)
    slots = [eng.new_sequence() for _ in range(batch)]
    ps = prompts(batch, PROMPT, cfg.vocab_size, 3)
    tok = torch.zeros(batch, dtype=torch.int32, device=eng.device)
    kernels.argmax(eng.step([StepEntry(s, p, [PROMPT - 1]) for s, p in zip(slots, ps)]), tok, batch)

    def one():
        kernels.argmax(eng.step([StepEntry(s, [0], [0]) for s in slots], device_tokens=tok), tok, batch)

    for _ in range(6):
        one()
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(3):
            one()
        torch.cuda.synchronize()
    ev = sorted((e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA),
                key=lambda e: e.time_range.start)
    last = ev[-(len(ev) // 3):]                      # the third step
    t0, prev_end = last[0].time_range.start, None
    print(f"decode step, batch {batch}, {layers} layers: start, end, added (us), kernel")
    for e in last:
        end = e.time_range.end
        added = end - (prev_end if prev_end is not None else e.time_range.start)
        prev_end = max(end, prev_end or end)
        print(f"{e.time_range.start - t0:9.2f} {end - t0:9.2f} {added:7.2f}  {e.name[:90]}")
    print(f"step: {prev_end - t0:.1f} us")


def main():
    global MODEL
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=int(os.environ.get("WORLD_SIZE", "1")))
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the configuration has (0: all)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--skip-points", action="store_true", help="leave out batch 1 and 64")
    ap.add_argument("--micro", default=None,
                    help="instead of the bench: gemm-decode, gemm-prefill (kernel microbenchmarks), timeline "
                         "(every kernel of one decode step with its start and end), sampler (a sampling step) or "
                         "sweep (decode steps at other batch sizes and context lengths)")
    ap.add_argument("--batch", type=int, default=BATCH, help="batch of --micro timeline")
    ap.add_argument("--model", default=MODEL, help="catalog entry whose layer sizes --micro sweep and timeline use")
    args = ap.parse_args()
    if args.micro:
        MODEL = args.model
    elif args.model != MODEL:
        print("bench.py: --model only applies to --micro runs; the bench line is for %s" % MODEL)
        return 2
    if args.micro == "timeline":
        timeline(args.batch, args.layers or 4)
        return 0
    if args.micro == "sampler":
        sampler_times()
        return 0
    if args.micro == "sweep":
        sweep(None if args.model == "qwen3-8b" else [(1, 1024), (8, 1024), (8, 8192), (64, 1024)])
        return 0
    if args.micro:
        micro(args.micro)
        return 0

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "xmiksay/rocml is a Rust + HIP (ROCm, gfx1101) workspace with no Python package; "
                          "it needs cargo, hipcc and a GGUF checkpoint, none of which exist here"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine works on one GPU; --gpus {args.gpus} is not supported")
        return 2
    steps, warmup = max(1, args.steps), max(3, args.warmup)

    import torch
    pk = peaks()
    max_slots = 64
    cfg, n_full, eng = build_engine(args.layers, max_tokens=max_slots * (PROMPT + 64 * 5), max_slots=max_slots)
    layers = cfg.num_hidden_layers
    vocab = cfg.vocab_size
    dev_gb = torch.cuda.memory_allocated() / 1e9

    prefill_ms = time_prefill(eng, vocab)
    pf = prefill_flops(cfg, layers, PREFILL_TOKENS)

    clocks = Clocks()
    clocks.start()
    ms, ctx_tokens, launched = time_decode(eng, BATCH, steps, warmup, vocab, seed=1)
    clk = clocks.stop()
    value = BATCH * 1000.0 / ms
    bytes_step = eng.model.weight_bytes_per_step() + ctx_tokens * eng.kv_bytes_per_token()
    achieved = bytes_step / (ms * 1e-3) / 1e9

    points = {}
    if not args.skip_points:
        for b in (1, 64):
            k = max(16, min(steps, 64))
            m, _, _ = time_decode(eng, b, k, warmup, vocab, seed=10 + b)
            points[f"decode_b{b}"] = round(b * 1000.0 / m, 1)

    e2e, h2d, d2h = e2e_decode(eng, BATCH, min(steps, 128), warmup, vocab)

    line = {
        "metric": "decode tok/s at batch 8 (Qwen3-8B layer sizes, bf16, random weights, prompts of 1024)",
        "value": round(value, 1), "unit": "tok/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: seeded uniform-random token ids, random-init weights",
        "config": {
            "model": "Qwen3-8B layer sizes", "layers": layers, "layers_full": n_full,
            "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
            "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": vocab,
            "tied_head": cfg.tie_word_embeddings, "global_batch": BATCH, "prompt_len": PROMPT,
            "seq_len": CTX, "decode_steps_timed": steps, "parallelism": "single GPU",
            "l2": "inputs larger than L2: every step reads all weights (GB: %.1f)" % (eng.model.weight_bytes_per_step() / 1e9),
            "device_gb": round(dev_gb, 1), "peaks": pk["source"],
        },
        "clocks": clk,
        "e2e": {"value": round(e2e, 1), "unit": "tok/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": launched,
        "prefill": {"value": round(PREFILL_TOKENS * 1000.0 / prefill_ms, 1), "tokens": PREFILL_TOKENS,
                    "ms": round(prefill_ms, 3), "frac": round(pf / (prefill_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
