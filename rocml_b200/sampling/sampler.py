"""Sampling a token for every sequence of a batch, on the GPU.

The host keeps what is sequential by nature, one xorshift64* stream per sequence, and hands
each step's uniform number to the kernel; the kernel does everything that touches the logits
(penalty, temperature, top-k, softmax, top-p, the walk).  Logits never leave the device; the
step's result is one int32 per sequence, read back through pinned memory.

Sampling is split into ``launch`` (enqueue the kernel and the copy back, return at once) and
``collect`` (wait for that copy, return the ids), so that a caller may enqueue the next step,
fed from ``PendingSample.device_tokens``, before it reads this one.  The pinned buffers form a
ring: a launch never writes host memory that an earlier launch's copies may still use.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

import numpy as np
import torch

from .. import kernels
from .params import SamplingParams, XorShift64Star


# one row's record as the kernel reads it (8 x 4 bytes)
_ROW = np.dtype([("temperature", "<f4"), ("top_k", "<i4"), ("top_p", "<f4"), ("u", "<f4"), ("penalty", "<f4"),
                 ("hist_begin", "<i4"), ("hist_len", "<i4"), ("pad", "<i4")])


@dataclass
class PendingSample:
    """A sampling step that has been enqueued.  ``device_tokens`` (int32, one per row) is valid
    for work enqueued after it on the same stream, until the next launch of the same sampler
    has run there."""

    n: int
    device_tokens: torch.Tensor
    host_tokens: torch.Tensor
    host_status: Optional[torch.Tensor]
    event: "torch.cuda.Event"


class Sampler:
    def __init__(self, device, max_batch: int = 256, max_window: int = 64, depth: int = 4):
        self.device = torch.device(device)
        self.max_batch = max_batch
        self.max_window = max_window
        self._ring = [{
            "rows": torch.zeros(max_batch * 8, dtype=torch.int32, pin_memory=True),
            "hist": torch.zeros(max_batch * max_window, dtype=torch.int32, pin_memory=True),
            "out": torch.zeros(max_batch, dtype=torch.int32, pin_memory=True),
            "status": torch.zeros(1, dtype=torch.int32, pin_memory=True),
            "event": None,
        } for _ in range(depth)]
        self._next = 0
        self._rows = torch.zeros(max_batch * 8, dtype=torch.int32, device=self.device)
        self._hist = torch.zeros(max_batch * max_window, dtype=torch.int32, device=self.device)
        self._out = torch.zeros(max_batch, dtype=torch.int32, device=self.device)

    def launch(self, logits: torch.Tensor, params: Sequence[SamplingParams],
               rngs: Sequence[Optional[XorShift64Star]], histories: Sequence[Sequence[int]],
               status: Optional[torch.Tensor] = None) -> PendingSample:
        """Enqueue one token per row of ``logits`` [n, V]; ``histories[i]`` is prompt + generated
        ids of row i (read only when its params have a repeat penalty).  ``status`` (a device
        int32) is copied back beside the tokens."""
        n = len(params)
        if n > self.max_batch:
            raise ValueError(f"{n} rows exceed the sampler's batch of {self.max_batch}")
        slot = self._ring[self._next]
        self._next = (self._next + 1) % len(self._ring)
        if slot["event"] is not None:
            slot["event"].synchronize()
        with torch.cuda.device(self.device):
            if all(p.is_greedy and p.repeat_penalty is None for p in params):
                kernels.argmax(logits, self._out, n)
            else:
                rec = slot["rows"].numpy().view(_ROW)
                hist = slot["hist"].numpy()
                key = tuple(map(id, params))
                if slot.get("key") != key:
                    # what does not change from step to step is written once per set of parameters
                    rec["temperature"][:n] = [float(p.temperature) for p in params]
                    rec["top_k"][:n] = [int(p.top_k or 0) for p in params]
                    rec["top_p"][:n] = [-1.0 if p.top_p is None else float(p.top_p) for p in params]
                    rec["penalty"][:n] = [0.0 if p.repeat_penalty is None else float(p.repeat_penalty) for p in params]
                    rec["hist_begin"][:n] = 0
                    rec["hist_len"][:n] = 0
                    slot["key"] = key
                    slot["params"] = list(params)        # keeps the ids alive, so that a key names one set only
                rec["u"][:n] = [0.0 if p.is_greedy else rngs[i].next_f32() for i, p in enumerate(params)]
                h_used = 0
                for i, p in enumerate(params):
                    if p.repeat_penalty is not None:
                        w = min(p.repeat_penalty_window, self.max_window)
                        tail = list(histories[i][-w:]) if w > 0 else []
                        hist[h_used:h_used + len(tail)] = tail
                        rec["hist_begin"][i], rec["hist_len"][i] = h_used, len(tail)
                        h_used += len(tail)
                self._rows[: n * 8].copy_(slot["rows"][: n * 8], non_blocking=True)
                if h_used:
                    self._hist[:h_used].copy_(slot["hist"][:h_used], non_blocking=True)
                kernels.sample(logits, n, self._rows, self._hist, self._out)
            slot["out"][:n].copy_(self._out[:n], non_blocking=True)
            if status is not None:
                slot["status"].copy_(status, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record()
            slot["event"] = ev
        return PendingSample(n, self._out, slot["out"], slot["status"] if status is not None else None, ev)

    @staticmethod
    def collect(pending: PendingSample) -> List[int]:
        """Wait for the step's ids and return them; raises if a kernel recorded a failure."""
        pending.event.synchronize()
        if pending.host_status is not None:
            kernels.raise_for_status(int(pending.host_status[0]))
        return pending.host_tokens[:pending.n].tolist()

    def sample(self, logits, params, rngs, histories) -> List[int]:
        return self.collect(self.launch(logits, params, rngs, histories))
