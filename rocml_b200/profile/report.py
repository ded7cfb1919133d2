"""A profile's records summed into a table: per phase, per kind of operation and per layer, the
time, its share, the achieved bytes and operations per second against the device's limits, the
least time the work could take (``t_min = max(bytes / bandwidth, flops / peak)``), the efficiency
``t_min / t`` and the time above the bound, by which the list of what to work on next is sorted.
The columns are the reference's (rocml/src/profile/report.rs:29-60, profile/human.rs:41-63).
"""
from __future__ import annotations

from typing import Dict, List


def _row(label, recs, phase_ms, peaks, dtype) -> Dict:
    ms = sum(r.ms for r in recs)
    nbytes = sum(r.nbytes for r in recs)
    flops = sum(r.flops for r in recs)
    sec = ms * 1e-3
    bw, fl = peaks.bytes_per_sec, peaks.flops_per_sec(dtype)
    t_min = max(nbytes / bw, flops / fl) * 1e3
    return {
        "label": label, "count": len(recs), "bytes": nbytes, "flops": flops, "elapsed_ms": ms,
        "gb_per_sec": nbytes / sec / 1e9 if sec > 0 else 0.0,
        "tflop_per_sec": flops / sec / 1e12 if sec > 0 else 0.0,
        "frac_of_bandwidth": nbytes / sec / bw if sec > 0 else 0.0,
        "frac_of_flops": flops / sec / fl if sec > 0 else 0.0,
        "pct_of_phase_time": 100.0 * ms / phase_ms if phase_ms > 0 else 0.0,
        "t_min_ms": t_min,
        "bound": "hbm" if nbytes / bw >= flops / fl else "flops",
        "efficiency": t_min / ms if ms > 0 else 0.0,
        "wasted_ms": ms - t_min,
    }


def build_report(prof) -> Dict:
    """JSON-ready: {"peaks", "phases": [{"phase", "steps", "step_ms", "ops_ms", "between_kernels_ms",
    "by_op", "by_layer"}], "worklist"}."""
    peaks, dtype = prof.peaks, prof.dtype
    phases = []
    order: List[str] = []
    for r in prof.ops:
        if r.phase not in order:
            order.append(r.phase)
    for phase in order:
        recs = [r for r in prof.ops if r.phase == phase]
        steps = [s for s in prof.steps if s.phase == phase]
        ops_ms = sum(r.ms for r in recs)
        step_ms = sum(s.ms for s in steps)
        by_op: Dict[str, list] = {}
        by_layer: Dict[str, list] = {}
        for r in recs:
            by_op.setdefault(r.op, []).append(r)
            by_layer.setdefault("(outside the layers)" if r.layer is None else f"layer {r.layer}", []).append(r)
        phases.append({
            "phase": phase, "steps": len(steps), "tokens": sum(s.n_tokens for s in steps),
            "step_ms": step_ms, "ops_ms": ops_ms, "between_kernels_ms": max(0.0, step_ms - ops_ms) if steps else 0.0,
            # steps whose launches the host had not all enqueued when the GPU was let go: their
            # kernels' times include the host's gaps
            "host_bound_steps": sum(1 for s in steps if s.gate_ms > 0 and s.host_ms > s.gate_ms),
            "total": _row("(all)", recs, ops_ms, peaks, dtype),
            "by_op": sorted((_row(k, v, ops_ms, peaks, dtype) for k, v in by_op.items()),
                            key=lambda x: -x["elapsed_ms"]),
            "by_layer": [_row(k, v, ops_ms, peaks, dtype) for k, v in by_layer.items()],
        })
    work = []
    for ph in phases:
        for row in ph["by_op"]:
            work.append((row["wasted_ms"], f"{ph['phase']} {row['label']}: {row['wasted_ms']:.3f} ms above its bound "
                         f"({row['elapsed_ms']:.3f} ms at {100 * row['efficiency']:.0f} % of the {row['bound']} limit, "
                         f"{row['pct_of_phase_time']:.1f} % of the phase)"))
    work.sort(key=lambda x: -x[0])
    return {
        "peaks": {"hbm_gbs": peaks.hbm_gbs, "tflops": peaks.flops_per_sec(dtype) / 1e12, "dtype": dtype,
                  "source": peaks.source},
        "phases": phases,
        "worklist": [w[1] for w in work[:8]],
    }


def to_human(report: Dict, layers: bool = False) -> str:
    pk = report["peaks"]
    out = [f"limits ({pk['source']}): {pk['hbm_gbs']:.0f} GB/s, {pk['tflops']:.0f} TFLOP/s {pk['dtype']}"]
    head = f"{'label':<30} {'n':>6} {'ms':>10} {'%time':>7} {'GB/s':>8} {'TFLOP/s':>8} {'%BW':>6} {'%FL':>6} {'t_min ms':>9} {'eff':>5} {'waste ms':>9}"

    def table(rows):
        lines = [head]
        for r in rows:
            lines.append(f"{r['label'][:30]:<30} {r['count']:>6} {r['elapsed_ms']:>10.3f} {r['pct_of_phase_time']:>6.1f}% "
                         f"{r['gb_per_sec']:>8.0f} {r['tflop_per_sec']:>8.1f} {100 * r['frac_of_bandwidth']:>5.1f}% "
                         f"{100 * r['frac_of_flops']:>5.1f}% {r['t_min_ms']:>9.3f} {r['efficiency']:>5.2f} {r['wasted_ms']:>9.3f}")
        return lines
    for ph in report["phases"]:
        out.append("")
        out.append(f"== {ph['phase']}: {ph['steps']} steps, {ph['tokens']} tokens, {ph['step_ms']:.3f} ms on the device, "
                   f"{ph['ops_ms']:.3f} ms in kernels, {ph['between_kernels_ms']:.3f} ms between them ==")
        if ph.get("host_bound_steps"):
            out.append(f"   ({ph['host_bound_steps']} of these steps took the host longer to enqueue than the GPU was "
                       "held back: their kernels' times include launch gaps)")
        out.append("-- by kind of operation --")
        out += table(ph["by_op"] + [ph["total"]])
        if layers:
            out.append("-- by layer --")
            out += table(ph["by_layer"])
    if report["worklist"]:
        out.append("")
        out.append("== what to work on (time above the bound) ==")
        out += report["worklist"]
    return "\n".join(out)
