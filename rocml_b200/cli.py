"""Command line: ``python -m rocml_b200 {generate,bench,models}``.

The commands, option names and meanings follow the reference's ``rocml-cli``
(rocml-cli/src/main.rs:26-38): ``--model <name-or-path>`` (common.rs:42-43), ``-n/--max-tokens``
(default 64, cmd_generate.rs:36-37), ``--ctx`` (cmd_generate.rs:41-42), ``-t/--temperature``,
``--top-p``, ``--top-k``, ``--seed`` with the precedence explicit flag > the named model's preset >
greedy (common.rs:147-176), and for ``bench`` ``--prompt-tokens`` 64, ``--decode-tokens`` 128,
``--runs`` 3, ``--depth``, ``--ctx``, ``--json`` (cmd_bench.rs:19-41); ``--profile`` prints the per-kernel
table against the device's limits after the run and ``--profile-json`` writes it
(cmd_generate.rs:47-48, cmd_bench.rs:43-57: only the last run is profiled).  Two things differ because
they lie outside this library: prompts are token ids (``--prompt-ids`` / ``--prompt-file`` /
``--prompt-len``; there is no tokenizer here), and ``--random`` generates seeded random weights for
a named size instead of downloading a checkpoint.  ``--dtype`` takes the place of ``--kv-cache``:
it selects the whole path (bfloat16 serving kernels, or true 32-bit).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import tempfile
import time
from typing import List, Optional

from .config import CATALOG, checkpoint_dir, config_from_dict, resolve
from .errors import RocmlError

DEFAULT_CTX = 4096   # when neither --ctx nor a preset gives one (rocml-cli/src/cmd_generate.rs:15-17)


def _model_args(p):
    p.add_argument("--model", required=True, help="a catalog name (see `models`) or a model folder")
    p.add_argument("--random", action="store_true",
                   help="for a catalog name: write seeded random weights of that size to a temporary folder")
    p.add_argument("--seed-weights", type=int, default=0, help="seed of --random")
    p.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    p.add_argument("--ctx", type=int, default=None, help="longest sequence the cache is sized for")


def _profile_args(p):
    p.add_argument("--profile", action="store_true",
                   help="time every kernel and print the table against the device's limits after the run")
    p.add_argument("--profile-json", default=None, metavar="PATH", help="write that table as JSON")
    p.add_argument("--profile-layers", action="store_true", help="with --profile: also the table by layer")


def _open_engine(args, batch: int, ctx: Optional[int] = None):
    from .engine import Engine
    from .weights import write_random_model
    resolved = resolve(args.model, must_exist=not args.random)
    entry = resolved.entry
    folder = resolved.path
    tmp = None
    if args.random:
        if entry is None:
            raise RocmlError("--random needs a catalog name (its sizes come from the catalog)")
        tmp = tempfile.TemporaryDirectory(prefix="rocml_b200_random_")
        folder = tmp.name
        print(f"writing random weights for {entry.name} to {folder} ...", file=sys.stderr, flush=True)
        write_random_model(folder, config_from_dict(entry.config), args.seed_weights)
    ctx = ctx or args.ctx or (entry.default_ctx if entry else DEFAULT_CTX)
    print(f"loading {args.model}... (ctx {ctx})", file=sys.stderr, flush=True)
    eng = Engine.from_folder(folder, dtype=args.dtype, max_tokens=batch * ((ctx + 63) // 64 * 64),
                             max_slots=max(batch, 1), max_seq_len=ctx)
    spec = eng.model.spec
    import torch
    free, total = torch.cuda.mem_get_info()
    print(f"loaded: {len(spec.schedule)} layers, hidden={spec.hidden}, vocab={spec.vocab}; "
          f"device memory free {free / 2**20:.0f} MiB / total {total / 2**20:.0f} MiB", file=sys.stderr, flush=True)
    return eng, entry, tmp


def _prompt_ids(args, vocab: int) -> List[int]:
    if args.prompt_ids:
        return [int(x) for x in args.prompt_ids.replace(",", " ").split()]
    if args.prompt_file:
        with open(args.prompt_file) as f:
            return [int(x) for x in f.read().replace(",", " ").split()]
    return synthetic_tokens(args.prompt_len, vocab, seed=0)


def synthetic_tokens(n: int, vocab: int, seed: int) -> List[int]:
    """Seeded uniform-random ids: content does not matter to a throughput run (the reference repeats
    a filler sentence for the same purpose, rocml-cli/src/cmd_bench.rs:249-255)."""
    import torch
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def _profiler(args, eng):
    if not (args.profile or args.profile_json):
        return None
    from .profile import Profiler
    return Profiler(eng.device, dtype=args.dtype)


def _emit_profile(args, prof):
    """The table on stdout (--profile), the same as JSON in a file (--profile-json).  Returns the report."""
    if prof is None:
        return None
    from .profile import to_human
    report = prof.report()
    if args.profile:
        print(to_human(report, layers=getattr(args, "profile_layers", False)))
    if args.profile_json:
        with open(args.profile_json, "w") as f:
            json.dump({"report": report}, f, indent=1)
        print(f"wrote profile JSON to {args.profile_json}", file=sys.stderr)
    return report


def roofline_of_run(eng, prompt_len: int, decode_tokens: int, batch: int, p_rate: float, d_rate: float, dtype: str):
    """What the measured rates are of the device's limits: the prompts' floating-point operations a
    second against the matrix peak, and the bytes a decode step has to read (every weight once, the
    live sequences' keys and values at the run's mean length) against the copy bandwidth."""
    from .profile import load_peaks
    peaks = load_peaks()
    _, p_flops = eng.model.step_cost([prompt_len] * batch, [prompt_len] * batch, batch)
    mean_ctx = prompt_len + (decode_tokens + 1) // 2
    d_bytes, _ = eng.model.step_cost([1] * batch, [mean_ctx] * batch, batch)
    p_frac = p_flops * (p_rate / (prompt_len * batch)) / peaks.flops_per_sec(dtype) if p_rate > 0 else 0.0
    d_gbs = d_bytes * (d_rate / batch) / 1e9 if d_rate > 0 else 0.0
    return {
        "peaks": peaks.source, "prefill_flops": p_flops, "prefill_frac_of_peak_flops": p_frac,
        "decode_bytes_per_step": d_bytes, "decode_gb_per_sec": d_gbs,
        "decode_frac_of_bandwidth": d_gbs / peaks.hbm_gbs,
    }


def cmd_generate(args) -> int:
    from .engine.generate import GenerateStats
    from .sampling import SamplingParams
    eng, entry, tmp = _open_engine(args, batch=1)
    preset = entry.sampling if entry else None
    base = SamplingParams() if preset is None else SamplingParams(preset.temperature, preset.top_k, preset.top_p, preset.seed)
    sampling = base.merged(args.temperature, args.top_k, args.top_p, args.seed)
    ids = _prompt_ids(args, eng.model.vocab)
    stats = GenerateStats()

    def show(_, tok):
        sys.stdout.write(f"{tok} ")
        sys.stdout.flush()
        return False

    prof = _profiler(args, eng)
    if prof is not None:
        with prof:
            out = eng.generate([ids], max_new_tokens=args.max_tokens, sampling=sampling, on_token=show, stats=stats,
                               run_ahead=False)
    else:
        out = eng.generate([ids], max_new_tokens=args.max_tokens, sampling=sampling, on_token=show, stats=stats)
    print()
    _emit_profile(args, prof)
    print(f"prompt: {stats.prompt_tokens} tokens in {stats.prefill_seconds:.3f}s "
          f"({stats.prompt_tokens_per_sec:.1f} tok/s); decode: {stats.decode_tokens} tokens in "
          f"{stats.decode_seconds:.3f}s ({stats.decode_tokens_per_sec:.1f} tok/s); finished: {out[0].finish_reason}",
          file=sys.stderr)
    return 0


def cmd_bench(args) -> int:
    from .engine.generate import GenerateStats
    if args.runs <= 0:
        raise RocmlError("--runs must be at least 1")
    prompt_len = args.depth if args.depth is not None else args.prompt_tokens
    need = prompt_len + args.decode_tokens
    eng, entry, tmp = _open_engine(args, batch=args.batch, ctx=args.ctx or need)
    vocab = eng.model.vocab
    prompts = [synthetic_tokens(prompt_len, vocab, seed=i) for i in range(args.batch)]
    eng.generate(prompts, max_new_tokens=2, stop_tokens=[], ignore_eos=True, max_batch=args.batch)   # warm-up
    p_rates, d_rates = [], []
    prof = None
    for run in range(args.runs):
        st = GenerateStats()
        eng.generate(prompts, max_new_tokens=args.decode_tokens, stop_tokens=[], ignore_eos=True,
                     max_batch=args.batch, stats=st)
        p_rates.append(st.prompt_tokens_per_sec)
        d_rates.append(st.decode_tokens_per_sec)
    p_med, d_med = statistics.median(p_rates), statistics.median(d_rates)
    prof = _profiler(args, eng)
    if prof is not None:
        # one more run, kernel by kernel: it does not count toward the medians (its steps run without
        # graphs and with events between the kernels)
        with prof:
            eng.generate(prompts, max_new_tokens=min(args.decode_tokens, 16), stop_tokens=[], ignore_eos=True,
                         max_batch=args.batch, run_ahead=False)
    roof = roofline_of_run(eng, prompt_len, args.decode_tokens, args.batch, p_med, d_med, args.dtype)
    if args.json:
        doc = {
            "model": args.model, "prompt_tokens": prompt_len, "decode_tokens": args.decode_tokens,
            "depth": args.depth, "runs": args.runs, "batch": args.batch, "dtype": args.dtype,
            "prompt_tokens_per_sec_median": p_med, "decode_tokens_per_sec_median": d_med,
            "roofline": roof,
        }
        if prof is not None:
            doc["profile"] = prof.report()
            if args.profile_json:
                _emit_profile(argparse.Namespace(profile=False, profile_json=args.profile_json), prof)
        print(json.dumps(doc))
    else:
        depth = f" @ depth {args.depth}" if args.depth is not None else ""
        print(f"prompt: {p_med:.1f} tok/s (median of {args.runs}, {100 * roof['prefill_frac_of_peak_flops']:.1f} % of the "
              f"{roof['peaks']} matrix peak); decode{depth}: {d_med:.1f} tok/s (median of {args.runs}, "
              f"{roof['decode_gb_per_sec']:.0f} GB/s, {100 * roof['decode_frac_of_bandwidth']:.1f} % of the "
              f"{roof['peaks']} copy bandwidth)")
        _emit_profile(args, prof)
    return 0


def cmd_models(_args) -> int:
    width = max(len(n) for n in CATALOG)
    root = checkpoint_dir()
    for name, e in CATALOG.items():
        path = os.path.join(root, e.folder)
        present = "present" if os.path.isfile(os.path.join(path, "config.json")) else "missing"
        print(f"{name:{width}}  {e.architecture:<18}  {present:<8}  {e.folder}")
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="rocml_b200", description=__doc__.split("\n\n")[0])
    sub = ap.add_subparsers(dest="command", required=True)

    g = sub.add_parser("generate", help="one completion for a prompt of token ids")
    _model_args(g)
    g.add_argument("--prompt-ids", default=None, help="token ids, comma or space separated")
    g.add_argument("--prompt-file", default=None, help="a file of token ids")
    g.add_argument("--prompt-len", type=int, default=16, help="length of a synthetic prompt when no ids are given")
    g.add_argument("-n", "--max-tokens", type=int, default=64)
    g.add_argument("-t", "--temperature", type=float, default=None)
    g.add_argument("--top-p", type=float, default=None)
    g.add_argument("--top-k", type=int, default=None)
    g.add_argument("--seed", type=int, default=None)
    _profile_args(g)
    g.set_defaults(fn=cmd_generate)

    b = sub.add_parser("bench", help="prompt and decode throughput, greedy, stop tokens ignored")
    _model_args(b)
    b.add_argument("--prompt-tokens", type=int, default=64)
    b.add_argument("--decode-tokens", type=int, default=128)
    b.add_argument("--runs", type=int, default=3)
    b.add_argument("--depth", type=int, default=None, help="prefill this many tokens instead of --prompt-tokens")
    b.add_argument("--batch", type=int, default=1, help="sequences decoded together")
    b.add_argument("--json", action="store_true")
    _profile_args(b)
    b.set_defaults(fn=cmd_bench)

    m = sub.add_parser("models", help="the catalog of model names, with present/missing")
    m.set_defaults(fn=cmd_models)

    args = ap.parse_args(argv)
    try:
        return args.fn(args)
    except RocmlError as e:
        print(f"error: {e}", file=sys.stderr)
        return 1


if __name__ == "__main__":
    sys.exit(main())
