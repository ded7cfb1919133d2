"""Timing of a step's kernels, one by one, with what each had to move and compute.

While a ``Profiler`` is active every kernel wrapper of ``rocml_b200.kernels`` brackets its launch
with a pair of CUDA events on the launching stream and files a record: the kernel's name, the
label and layer its callers set (``scope``), the step's phase, and the bytes and operations of
``cost``.  The engine runs such steps without CUDA graphs, and holds the GPU back behind a short
spin kernel while the host enqueues a step, so that the kernels then run back to back and a
record's time is the kernel's own, not the host's launch gap.  Events between kernels keep a
kernel from starting under its predecessor's tail (programmatic dependent launch), so a profiled
step is somewhat slower than a served one; ``StepRecord`` keeps both ends of the step for that
comparison.

The reference does the same with HIP event pairs around each operation of its forward pass
(rocml/src/profile/mod.rs:163-252) and resolves them when the run is over.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch

from .peaks import Peaks, load_peaks

ACTIVE: Optional["Profiler"] = None


class _Null:
    def __enter__(self):
        return None

    def __exit__(self, *exc):
        return False


_NULL = _Null()


def scope(**tags):
    """``with scope(layer=3):`` / ``with scope(op="o_proj"):`` tags the kernels launched inside;
    free when no profiler is active."""
    p = ACTIVE
    return _NULL if p is None else _Scope(p, tags)


class _Scope:
    def __init__(self, prof, tags):
        self.prof, self.tags = prof, tags

    def __enter__(self):
        self.prof._stack.append(self.tags)

    def __exit__(self, *exc):
        self.prof._stack.pop()
        return False


@dataclass
class OpRecord:
    kernel: str
    op: str
    layer: Optional[int]
    phase: str
    nbytes: int
    flops: int
    start: object = None
    end: object = None
    ms: float = 0.0


@dataclass
class StepRecord:
    phase: str
    n_tokens: int
    n_seqs: int
    start: object = None
    end: object = None
    ms: float = 0.0
    first_op: int = 0
    n_ops: int = 0
    host_ms: float = 0.0      # what the host took to enqueue the step
    gate_ms: float = 0.0      # how long the GPU was held back meanwhile; host_ms beyond it shows in the kernels' times


@dataclass
class StepFacts:
    """What the cost of an attention kernel depends on and only the host knows."""
    q_lens: List[int] = field(default_factory=list)
    kv_lens: List[int] = field(default_factory=list)


class Profiler:
    def __init__(self, device="cuda:0", peaks: Optional[Peaks] = None, dtype: str = "bfloat16", gate_ms: float = 20.0):
        self.device = torch.device(device)
        self.peaks = peaks or load_peaks()
        self.dtype = dtype
        self.gate_ms = float(gate_ms)
        self.ops: List[OpRecord] = []
        self.steps: List[StepRecord] = []
        self.facts = StepFacts()
        self._stack: List[Dict] = []
        self._open_step: Optional[StepRecord] = None
        self._depth = 0
        self._last_end = None
        self._last_end_launches = -1
        self._host_ms: Dict[str, float] = {}      # per phase: the longest a step took to enqueue so far

    # ---- switching on and off ------------------------------------------------------------------
    def __enter__(self):
        global ACTIVE
        if ACTIVE is not None:
            raise RuntimeError("a profiler is already active")
        ACTIVE = self
        return self

    def __exit__(self, *exc):
        global ACTIVE
        ACTIVE = None
        return False

    def scope(self, **tags):
        return _Scope(self, tags)

    # ---- a step ----------------------------------------------------------------------------------
    def step(self, phase: str, q_lens, kv_lens):
        """``with prof.step("decode", q_lens, kv_lens):`` around everything a step enqueues.  Nested
        uses (the sampling around the model's pass) belong to the outermost."""
        return _Step(self, phase, list(q_lens), list(kv_lens))

    def _gate(self, phase: str) -> float:
        """A spin on the stream while the host enqueues the step's launches: gate_ms for the first step
        of a phase, then one and a half times the longest enqueue seen (at most a second)."""
        if self.gate_ms <= 0 or self.device.type != "cuda":
            return 0.0
        from .. import kernels
        ms = min(1000.0, max(self.gate_ms, 1.5 * self._host_ms.get(phase, 0.0)))
        kernels.hold(ms * 1e3)
        return ms

    # ---- a kernel ----------------------------------------------------------------------------------
    def begin(self):
        from .. import kernels
        if self._last_end is not None and self._last_end_launches == kernels.launch_count:
            return self._last_end           # nothing ran since the last record ended: share the event
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        return ev

    def end(self, start, kernel: str, nbytes: int, flops: int):
        from .. import kernels
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        tags = {}
        for t in self._stack:
            tags.update(t)
        phase = self._open_step.phase if self._open_step is not None else tags.get("phase", "other")
        self.ops.append(OpRecord(kernel, tags.get("op") or kernel, tags.get("layer"), phase, int(nbytes), int(flops),
                                 start, ev))
        self._last_end, self._last_end_launches = ev, kernels.launch_count

    # ---- when the run is over ------------------------------------------------------------------------
    def finish(self):
        """Wait for the device and turn the events into milliseconds."""
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        for r in self.ops:
            if r.start is not None:
                r.ms = r.start.elapsed_time(r.end)
                r.start = r.end = None
        for s in self.steps:
            if s.start is not None:
                s.ms = s.start.elapsed_time(s.end)
                s.start = s.end = None
        self._last_end = None
        return self

    def report(self):
        from .report import build_report
        return build_report(self.finish())


class _Step:
    def __init__(self, prof: Profiler, phase, q_lens, kv_lens):
        self.prof, self.phase, self.q_lens, self.kv_lens = prof, phase, q_lens, kv_lens

    def __enter__(self):
        p = self.prof
        p._depth += 1
        if p._depth > 1:
            if self.q_lens:
                p.facts = StepFacts(self.q_lens, self.kv_lens)
                if p._open_step is not None and p._open_step.n_seqs == 0:
                    p._open_step.n_tokens, p._open_step.n_seqs = sum(self.q_lens), len(self.q_lens)
            return None
        p.facts = StepFacts(self.q_lens, self.kv_lens)
        rec = StepRecord(self.phase, sum(self.q_lens), len(self.q_lens), first_op=len(p.ops))
        p._last_end = None                      # the first kernel's time starts at the step, not at the last step's end
        rec.gate_ms = p._gate(self.phase)
        self._t0 = time.perf_counter()
        rec.start = torch.cuda.Event(enable_timing=True)
        rec.start.record()
        p._open_step = rec
        return rec

    def __exit__(self, *exc):
        p = self.prof
        p._depth -= 1
        if p._depth:
            return False
        rec = p._open_step
        rec.end = torch.cuda.Event(enable_timing=True)
        rec.end.record()
        rec.host_ms = (time.perf_counter() - self._t0) * 1e3
        p._host_ms[rec.phase] = max(p._host_ms.get(rec.phase, 0.0), rec.host_ms)
        rec.n_ops = len(p.ops) - rec.first_op
        p.steps.append(rec)
        p._open_step = None
        return False
