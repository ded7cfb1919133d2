"""Measurements of the engine on one GPU: the pieces ``bench.py`` prints its line from, the other
workloads of the same kind, and the sweeps and timelines that the notes under ``profiles/`` quote.

    python -m rocml_b200.measure sweep [--model NAME]         decode steps over batch sizes and contexts
    python -m rocml_b200.measure timeline [--batch B]         every kernel of one decode step, start and end
    python -m rocml_b200.measure timeline --prompt N          the same for the step that takes a prompt of N tokens
    python -m rocml_b200.measure sampler                      one sampling step, by way of sampling and batch
    python -m rocml_b200.measure gemm-decode | gemm-prefill   the tensor-core product alone, in a CUDA graph
    python -m rocml_b200.measure workload 4b-long | 32b       a whole generation through Engine.generate
    python -m rocml_b200.measure float32                      the 32-bit path at the benchmark's layer sizes
    python -m rocml_b200.measure profile [--dtype float32]    the per-kernel table of --profile, random weights
    python -m rocml_b200.measure host [--model NAME]          what the Python host costs a decode step

Everything is timed on the device with CUDA events after warm-up; weights are random, token ids
seeded uniform-random (the reference's bench repeats a filler sentence for the same purpose,
rocml-cli/src/cmd_bench.rs:249-255, and reports the median of its runs, :257-265).
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

MODEL = "qwen3-8b"          # catalog entry with the benchmark's layer sizes
PROMPT = 1024
PREFILL_TOKENS = 2048
CTX = 4096
BATCH = 8


def peaks():
    from .profile import load_peaks
    p = load_peaks()
    return {"hbm_gbs": p.hbm_gbs, "bf16_tflops": p.bf16_tflops, "bf16_tflops_sustained": p.bf16_tflops_sustained,
            "f32_tflops": p.f32_tflops, "source": p.source}


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


def build_engine(layers, max_tokens, max_slots, model=None, dtype="bfloat16", ctx=None):
    """An engine with random weights of a catalog entry's layer sizes (``layers`` of its layers; 0: all)."""
    import torch
    from .config import CATALOG, config_from_dict
    from .engine import Engine, Model
    from .parts import BuildEnv

    full = dict(CATALOG[model or MODEL].config)
    n_full = full["num_hidden_layers"]
    if layers:
        full["num_hidden_layers"] = layers
    cfg = config_from_dict(full)
    dev = torch.device("cuda:0")
    with torch.cuda.device(dev):
        m = Model(cfg.to_model_spec(), BuildEnv(dev, torch.float32 if dtype == "float32" else torch.bfloat16))
        m.load_random(seed=0)
        eng = Engine(m, max_tokens=max_tokens, max_slots=max_slots, max_step_tokens=4096, max_seq_len=ctx or CTX)
    return cfg, n_full, eng


def prompts(n, length, vocab, seed):
    import torch
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n, length), generator=g).tolist()


def time_decode(eng, batch, steps, warmup, vocab, seed):
    """K decode steps of `batch` sequences after prompts of PROMPT tokens, timed with CUDA events.
    Returns (ms per step, mean cache tokens read per step, kernels launched in the timed region)."""
    import torch
    from . import StepEntry, kernels
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
    from . import StepEntry, kernels
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


def prefill_flops(eng, T):
    """Floating-point operations of one prompt of T tokens with logits at its last place, asked of the
    model's parts (products and causal attention)."""
    return eng.model.step_cost([T], [T], 1)[1]


def e2e_decode(eng, batch, steps, warmup, vocab):
    """Decoded tokens per second through Engine.generate: host token ids in, host token ids out,
    a pinned-memory copy each way in every step."""
    from . import GenerateStats
    ps = prompts(batch, PROMPT, vocab, 7)
    eng.generate(ps, max_new_tokens=max(warmup, 2), stop_tokens=[], ignore_eos=True, max_batch=batch)
    stats = GenerateStats()
    eng.generate(ps, max_new_tokens=steps + 1, stop_tokens=[], ignore_eos=True, max_batch=batch, stats=stats)
    return stats.decode_tokens / stats.decode_seconds, eng.last_h2d_bytes, batch * 4


def micro(which, model=None):
    """Kernel microbenchmarks: each kernel launched back to back inside a CUDA graph (no host
    time), at the Qwen3-8B layer sizes.  Results are printed, one line per case; they feed the
    notes under profiles/ and are not part of the bench line."""
    import torch
    from . import kernels
    from .config import CATALOG, config_from_dict
    cfg = config_from_dict(CATALOG[model or MODEL].config)
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
        raise SystemExit(f"unknown product measurement {which!r}: gemm-decode or gemm-prefill")


def sampler_times():
    """Time of one sampling step (kernel, copy of the ids to the host, the host's own part) over logits of the
    benchmark's vocabulary, for the ways of sampling and a few batch sizes; beside it the kernel's own time,
    launched back to back."""
    import torch
    from .config import CATALOG, config_from_dict
    from .sampling import Sampler, SamplingParams
    from .sampling.params import XorShift64Star
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
            from . import kernels
            run = (lambda: kernels.argmax(logits, s._out, batch)) if sp.is_greedy else \
                (lambda: kernels.sample(logits, batch, s._rows, s._hist, s._out))
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(20):
                run()
            b.record()
            torch.cuda.synchronize()
            print(f"batch {batch:3d}  {name:40s} {wall:8.1f} us a step, kernel {a.elapsed_time(b) / 20 * 1e3:7.1f} us")


def sweep(cases=None, steps=32, model=None):
    """Decode steps at other batch sizes and context lengths than the bench line's: milliseconds a step,
    tokens a second, and the bytes a step has to read (weights once, the live cache) over its time, as a
    fraction of the measured copy bandwidth.  All layers of the configuration; prompts are fed in pieces
    of at most 4,096 tokens."""
    import torch
    from . import StepEntry, kernels
    cases = cases or [(1, 1024), (1, 8192), (1, 32000), (4, 16000), (8, 1024), (8, 8192), (8, 32000), (16, 2048),
                      (32, 1024), (32, 8192), (64, 1024), (64, 4000), (128, 1024), (256, 1024)]
    pk = peaks()
    print("batch  context  ms/step    tok/s   GB/step   GB/s  of %s copy bandwidth" % pk["source"])
    for batch, ctx in cases:
        cfg, n_full, eng = build_engine(0, batch * ((ctx + 256 + 63) // 64 * 64), batch, model=model, ctx=ctx + 256)
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


def prompt_timeline(n_tokens, layers=4, model=None):
    """The same listing for the step that takes one prompt of ``n_tokens`` tokens (no CUDA graph: a prompt's
    kernels are long enough that the host stays ahead of them)."""
    import torch
    from torch.profiler import ProfilerActivity, profile
    from . import StepEntry
    cfg, n_full, eng = build_engine(layers, n_tokens + 256, 1, model=model)
    p = prompts(1, n_tokens, cfg.vocab_size, 3)[0]

    def one():
        slot = eng.new_sequence()
        eng.step([StepEntry(slot, p, [n_tokens - 1])])
        eng.release(slot)

    for _ in range(3):
        one()
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(3):
            one()
        torch.cuda.synchronize()
    ev = sorted((e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA),
                key=lambda e: e.time_range.start)
    last = ev[-(len(ev) // 3):]
    t0, prev_end = last[0].time_range.start, None
    print(f"one prompt of {n_tokens} tokens, {layers} layers: start, end, added (us), kernel")
    for e in last:
        end = e.time_range.end
        added = end - (prev_end if prev_end is not None else e.time_range.start)
        prev_end = max(end, prev_end or end)
        print(f"{e.time_range.start - t0:9.2f} {end - t0:9.2f} {added:7.2f}  {e.name[:90]}")
    print(f"step: {prev_end - t0:.1f} us")


def timeline(batch=BATCH, layers=4, model=None):
    """Where a decode step's time goes, kernel by kernel, as the step really runs (inside its CUDA
    graph, kernels overlapping their predecessors through programmatic dependent launch): start and
    end of every kernel from the profiler's activity records (CUPTI, no kernel is replayed), and for
    each kernel the time from its predecessor's end to its own end, which is what it adds to the step."""
    import torch
    from torch.profiler import ProfilerActivity, profile
    from . import StepEntry, kernels
    cfg, n_full, eng = build_engine(layers, batch * (PROMPT + 256), batch, model=model)
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




# ---- whole generations through the entry point ------------------------------------------------------------

WORKLOADS = {
    # name: (catalog entry, context, batch, what the prompts are, new tokens, sampling)
    "4b-long": dict(model="qwen3-4b", ctx=32768, prompts=[30000, 8000, 1000, 17], new_tokens=128,
                    sampling=(0.6, 20, 0.95)),
    "32b": dict(model="qwen3-32b", ctx=2048, prompts=("uniform", 64, 64, 1024), new_tokens=None, sampling=None),
}


def workload(name, layers=0, runs=1):
    """One of the larger workloads, whole, through ``Engine.generate`` (host token ids in and out):

    * ``4b-long``: Qwen3-4B layer sizes, a cache of 32,768 tokens a sequence, a batch of four prompts of
      30000 / 8000 / 1000 / 17 tokens, then 128 tokens each at temperature 0.6, top-k 20, top-p 0.95;
    * ``32b``: Qwen3-32B layer sizes (65.5 GB of weights), 64 prompts of lengths uniform in [64, 1024],
      greedy until every sequence holds 2,048 tokens: the shorter a prompt, the longer it decodes,
      and the batch shrinks as sequences fill up.

    Returns a JSON-ready record: prompt and decode tokens a second, the bytes a decode step has to read
    on average (every weight once and the live sequences' keys and values) and what that is of the
    copy bandwidth, the prompts' operations a second and what that is of the matrix peak."""
    import torch
    from . import GenerateStats, SamplingParams
    w = WORKLOADS[name]
    pk = peaks()
    if w["prompts"][0] == "uniform":
        _, n, lo, hi = w["prompts"]
        g = torch.Generator().manual_seed(32)
        lens = torch.randint(lo, hi + 1, (n,), generator=g).tolist()
    else:
        lens = list(w["prompts"])
    batch, ctx = len(lens), w["ctx"]
    cfg, n_full, eng = build_engine(layers, batch * ((ctx + 63) // 64 * 64), batch, model=w["model"], ctx=ctx)
    g = torch.Generator().manual_seed(5)
    ps = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in lens]
    sp = SamplingParams(*w["sampling"][:1], top_k=w["sampling"][1], top_p=w["sampling"][2], seed=0) if w["sampling"] \
        else SamplingParams()
    from .engine.generate import Request, generate
    news = [w["new_tokens"] if w["new_tokens"] is not None else ctx - n for n in lens]
    reqs = [Request(p, k, sp, [], True) for p, k in zip(ps, news)]
    # warm-up: the same prompts with a few new tokens (loads every kernel, captures the first graphs)
    generate(eng, [Request(p, 3, sp, [], True) for p in ps], max_batch=batch)
    out = []
    for _ in range(max(1, runs)):
        st = GenerateStats()
        torch.cuda.synchronize()
        done = generate(eng, reqs, max_batch=batch, stats=st)
        torch.cuda.synchronize()
        assert [len(c.tokens) for c in done] == news
        # bytes the decode steps had to read: step k (1-based) runs the sequences that still want a
        # token, each 'prompt + k' long afterwards
        kvb, wb = eng.kv_bytes_per_token(), eng.model.weight_bytes_per_step()
        total = 0
        for k in range(1, max(news)):
            live = [n + k for n, m in zip(lens, news) if m > k]
            total += wb + kvb * sum(live)
        steps = max(news) - 1
        _, pflops = eng.model.step_cost(lens, lens, batch)
        gbs = total / st.decode_seconds / 1e9
        out.append({
            "prefill_tok_s": st.prompt_tokens_per_sec, "prefill_s": st.prefill_seconds,
            "prefill_tflops": pflops / st.prefill_seconds / 1e12,
            "prefill_frac": pflops / st.prefill_seconds / (pk["bf16_tflops"] * 1e12),
            "decode_tok_s": st.decode_tokens_per_sec, "decode_s": st.decode_seconds, "decode_steps": steps,
            "decode_tokens": st.decode_tokens, "gb_per_step": total / steps / 1e9, "gb_per_s": gbs,
            "decode_frac": gbs / pk["hbm_gbs"],
        })
    best = sorted(out, key=lambda r: r["decode_s"])[len(out) // 2]
    rec = {"workload": name, "model": w["model"] + " layer sizes", "layers": cfg.num_hidden_layers, "layers_full": n_full,
           "batch": batch, "ctx": ctx, "prompt_tokens": sum(lens), "prompt_lens": lens if batch <= 8 else
           f"uniform in [{min(lens)}, {max(lens)}], mean {sum(lens) / batch:.0f}",
           "sampling": "temperature %.1f top-k %d top-p %.2f" % w["sampling"] if w["sampling"] else "greedy",
           "runs": len(out), "peaks": pk["source"], "device_gb": round(torch.cuda.memory_allocated() / 1e9, 1)}
    rec.update({k: (round(v, 4) if isinstance(v, float) else v) for k, v in best.items()})
    return rec


def float32_point(layers=4, steps=16, warmup=3):
    """The true 32-bit path at the benchmark's layer sizes (``layers`` of its layers): decode at batch 8
    after prompts of 1,024 tokens, and one prompt of 2,048 tokens.  The decode step is read against
    the copy bandwidth (32-bit weights: twice the bytes), the prompt against the CUDA cores' nominal
    32-bit rate."""
    import torch
    pk = peaks()
    cfg, n_full, eng = build_engine(layers, 8 * (PROMPT + 64 * 3) + PREFILL_TOKENS + 64, 9, dtype="float32")
    pre_ms = time_prefill(eng, cfg.vocab_size, runs=2, warmup=1)
    ms, ctx_tokens, _ = time_decode(eng, BATCH, steps, warmup, cfg.vocab_size, seed=2)
    nbytes = eng.model.weight_bytes_per_step() + ctx_tokens * eng.kv_bytes_per_token()
    flops = prefill_flops(eng, PREFILL_TOKENS)
    rec = {"layers": layers, "layers_full": n_full, "decode_b8_tok_s": round(BATCH * 1e3 / ms, 1), "decode_ms": round(ms, 3),
           "decode_frac_hbm": round(nbytes / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], 4),
           "prefill_tok_s": round(PREFILL_TOKENS * 1e3 / pre_ms, 1), "prefill_ms": round(pre_ms, 2),
           "prefill_tflops": round(flops / (pre_ms * 1e-3) / 1e12, 2),
           "prefill_frac_f32": round(flops / (pre_ms * 1e-3) / (pk["f32_tflops"] * 1e12), 4)}
    del eng
    torch.cuda.empty_cache()
    return rec


def profile_table(model=None, layers=0, batch=BATCH, dtype="bfloat16", prompt=PROMPT, steps=8, by_layer=False):
    """The per-kernel table of ``--profile`` for prompts of ``prompt`` tokens and ``steps`` decode steps
    at a catalog entry's layer sizes, random weights made on the device."""
    from . import StepEntry
    from .profile import Profiler, to_human
    cfg, n_full, eng = build_engine(layers, batch * (prompt + 64 * 2), batch, model=model, dtype=dtype)
    ps = prompts(batch, prompt + steps, cfg.vocab_size, 3)

    def run():
        slots = [eng.new_sequence() for _ in ps]
        eng.step([StepEntry(s, p[:prompt], [prompt - 1]) for s, p in zip(slots, ps)])
        for t in range(steps):
            eng.step([StepEntry(s, [p[prompt + t]], [0]) for s, p in zip(slots, ps)])
        for s in slots:
            eng.release(s)
    run()
    with Profiler(eng.device, dtype=dtype) as prof:
        run()
    print(f"{model or MODEL} layer sizes, {cfg.num_hidden_layers} of {n_full} layers, {dtype}, batch {batch}, "
          f"prompts of {prompt} tokens, {steps} decode steps")
    print(to_human(prof.report(), layers=by_layer))


def host_cost(model=None, layers=0, batches=(1, 8, 64), steps=64):
    """What the Python host costs a decode step: the step on the device alone (CUDA events around steps
    whose tokens never leave the device), the same through ``Engine.generate`` with the loop reading
    every step before it enqueues the next, and with the loop running one step ahead (the default),
    in milliseconds a step; and the host's own time for one step's bookkeeping, packing and launch."""
    import torch
    from . import GenerateStats, StepEntry
    cfg, n_full, eng = build_engine(layers, 64 * (PROMPT + 64 * 4), 64, model=model)
    print(f"{model or MODEL} layer sizes, {cfg.num_hidden_layers} layers: milliseconds a decode step")
    print("batch   device   generate, step by step   generate, one step ahead   host work a step")
    for b in batches:
        dev_ms, _, _ = time_decode(eng, b, steps, 4, cfg.vocab_size, seed=b)
        ps = prompts(b, PROMPT, cfg.vocab_size, 7)
        out = {}
        for ahead in (False, True):
            eng.generate(ps, max_new_tokens=4, stop_tokens=[], ignore_eos=True, max_batch=b, run_ahead=ahead)
            best = None
            for _ in range(3):
                st = GenerateStats()
                eng.generate(ps, max_new_tokens=steps + 1, stop_tokens=[], ignore_eos=True, max_batch=b, stats=st,
                             run_ahead=ahead)
                ms = st.decode_seconds / steps * 1e3
                best = ms if best is None else min(best, ms)
            out[ahead] = best
        # the host's part alone: bookkeeping, packing and enqueueing of a step while the GPU is held busy
        # (three steps at a time: the ring of pinned buffers lets the host run four steps ahead)
        slots = [eng.new_sequence() for _ in range(b)]
        eng.step([StepEntry(s, p, [PROMPT - 1]) for s, p in zip(slots, ps)])
        tok = torch.zeros(b, dtype=torch.int32, device=eng.device)
        eng.step([StepEntry(s, [0], [0]) for s in slots], device_tokens=tok)
        from . import kernels
        host = []
        for _ in range(8):
            torch.cuda.synchronize()
            kernels.hold(20e3)                                # the GPU is busy for 20 ms
            t0 = time.perf_counter()
            for _ in range(3):
                eng.step([StepEntry(s, [0], [0]) for s in slots], device_tokens=tok)
            host.append((time.perf_counter() - t0) / 3 * 1e3)
        host_ms = statistics.median(host)
        torch.cuda.synchronize()
        for s in slots:
            eng.release(s)
        print(f"{b:5d} {dev_ms:8.3f} {out[False]:24.3f} {out[True]:26.3f} {host_ms:18.3f}", flush=True)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m rocml_b200.measure", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("what", choices=["sweep", "timeline", "sampler", "gemm-decode", "gemm-prefill", "workload", "float32",
                                     "profile", "host"])
    ap.add_argument("name", nargs="?", default=None, help="for workload: " + " or ".join(WORKLOADS))
    ap.add_argument("--model", default=MODEL, help="catalog entry whose layer sizes are used")
    ap.add_argument("--batch", type=int, default=BATCH, help="batch of timeline")
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the entry has (0: all; timeline: 4)")
    ap.add_argument("--runs", type=int, default=1)
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"], help="of profile")
    ap.add_argument("--prompt", type=int, default=PROMPT, help="prompt length of profile; of timeline: list a prompt's step instead")
    args = ap.parse_args(argv)
    if args.what == "sweep":
        sweep(None if args.model == "qwen3-8b" else [(1, 1024), (8, 1024), (8, 8192), (64, 1024)], model=args.model)
    elif args.what == "timeline":
        if args.prompt != PROMPT:
            prompt_timeline(args.prompt, args.layers or 4, model=args.model)
        else:
            timeline(args.batch, args.layers or 4, model=args.model)
    elif args.what == "sampler":
        sampler_times()
    elif args.what in ("gemm-decode", "gemm-prefill"):
        micro(args.what, model=args.model)
    elif args.what == "float32":
        print(json.dumps(float32_point(args.layers or 4)))
    elif args.what == "host":
        host_cost(args.model, args.layers)
    elif args.what == "profile":
        profile_table(args.model, args.layers, args.batch, args.dtype, args.prompt)
    else:
        if args.name not in WORKLOADS:
            ap.error("workload needs one of: " + ", ".join(WORKLOADS))
        print(json.dumps(workload(args.name, args.layers, args.runs)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
