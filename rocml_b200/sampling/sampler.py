"""Sampling a token for every sequence of a batch, on the GPU.

The host keeps what is sequential by nature, one xorshift64* stream per sequence, and hands
each step's uniform number to the kernel; the kernel does everything that touches the logits
(penalty, temperature, top-k, softmax, top-p, the walk).  Logits never leave the device; the
step's result is one int32 per sequence, read back through pinned memory.
"""
from __future__ import annotations

import struct
from typing import List, Optional, Sequence

import numpy as np
import torch

from .. import kernels
from .params import SamplingParams, XorShift64Star


class Sampler:
    def __init__(self, device, max_batch: int = 256, max_window: int = 64):
        self.device = torch.device(device)
        self.max_batch = max_batch
        self.max_window = max_window
        self._rows_host = torch.zeros(max_batch * 8, dtype=torch.int32, pin_memory=True)
        self._rows = torch.zeros(max_batch * 8, dtype=torch.int32, device=self.device)
        self._hist_host = torch.zeros(max_batch * max_window, dtype=torch.int32, pin_memory=True)
        self._hist = torch.zeros(max_batch * max_window, dtype=torch.int32, device=self.device)
        self._out = torch.zeros(max_batch, dtype=torch.int32, device=self.device)
        self._out_host = torch.zeros(max_batch, dtype=torch.int32, pin_memory=True)

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams],
               rngs: Sequence[Optional[XorShift64Star]], histories: Sequence[Sequence[int]]) -> List[int]:
        """One token per row of ``logits`` [n, V]; ``histories[i]`` is prompt + generated ids of
        row i (read only when its params have a repeat penalty)."""
        n = len(params)
        if n > self.max_batch:
            raise ValueError(f"{n} rows exceed the sampler's batch of {self.max_batch}")
        with torch.cuda.device(self.device):
            if all(p.is_greedy and p.repeat_penalty is None for p in params):
                kernels.argmax(logits, self._out, n)
            else:
                rows = self._rows_host.numpy()
                hist = self._hist_host.numpy()
                h_used = 0
                for i, p in enumerate(params):
                    u = 0.0 if p.is_greedy else rngs[i].next_f32()
                    pen, hb, hl = 0.0, 0, 0
                    if p.repeat_penalty is not None:
                        w = min(p.repeat_penalty_window, self.max_window)
                        tail = list(histories[i][-w:]) if w > 0 else []
                        hb, hl = h_used, len(tail)
                        hist[hb:hb + hl] = tail
                        h_used += hl
                        pen = float(p.repeat_penalty)
                    rec = struct.pack("<fifffiii", float(p.temperature), int(p.top_k or 0),
                                      -1.0 if p.top_p is None else float(p.top_p), u, pen, hb, hl, 0)
                    rows[i * 8:(i + 1) * 8] = np.frombuffer(rec, dtype=np.int32)
                self._rows[: n * 8].copy_(self._rows_host[: n * 8], non_blocking=True)
                if h_used:
                    self._hist[:h_used].copy_(self._hist_host[:h_used], non_blocking=True)
                kernels.sample(logits, n, self._rows, self._hist, self._out)
            self._out_host[:n].copy_(self._out[:n], non_blocking=True)
            torch.cuda.current_stream().synchronize()
        return self._out_host[:n].tolist()
