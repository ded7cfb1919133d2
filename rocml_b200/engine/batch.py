"""The tokens of one step, as the kernels see them.

A step carries tokens of several sequences packed one after another.  Per token: its id,
its absolute position in its sequence, and its sequence's slot (-1 marks padding, which
every kernel skips).  Per sequence: its slot, where its tokens start (``cu_q``) and how
long it is once this step's tokens are appended (``kv_len``).  The integers travel to the
device in ONE copy from pinned host memory; the device tensors are views of one buffer
whose address does not change, so a captured CUDA graph can be replayed on new contents.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import numpy as np
import torch


@dataclass
class HostBatch:
    """The same facts on the host, for parts that are not written as kernels (test toys)."""

    seq_slots: List[int]
    q_lens: List[int]
    kv_lens: List[int]
    want_rows: List[int]


class BatchBuffers:
    """Fixed-capacity integer storage for a step's metadata: one device buffer, and a ring of
    pinned host buffers in front of it so that filling the next step's integers never
    overwrites a copy that is still in flight."""

    def __init__(self, max_tokens: int, max_seqs: int, max_want: int, device, depth: int = 4):
        self.max_tokens, self.max_seqs, self.max_want = max_tokens, max_seqs, max_want
        sizes = [max_tokens, max_tokens, max_tokens, max_seqs, max_seqs + 1, max_seqs, max_want]
        self._offsets = np.concatenate([[0], np.cumsum(sizes)]).astype(np.int64)
        total = int(self._offsets[-1])
        self.device = torch.device(device)
        self._cuda = self.device.type == "cuda"
        self._hosts = [torch.zeros(total, dtype=torch.int32, pin_memory=self._cuda) for _ in range(depth)]
        self._events = [None] * depth
        self._next = 0
        self.dev = torch.zeros(total, dtype=torch.int32, device=device)

    def _d(self, i):
        return self.dev[int(self._offsets[i]):int(self._offsets[i + 1])]

    def fill(self, token_ids, positions, slot_of_token, cu_q, kv_len, want_rows, seq_slot,
             pad_tokens: int, pad_seqs: int, pad_want: int) -> None:
        """Write one step's integers (padded to the given counts) and copy them to the device."""
        T, B, W = len(token_ids), len(seq_slot), len(want_rows)
        if pad_tokens > self.max_tokens or pad_seqs > self.max_seqs or pad_want > self.max_want:
            raise ValueError("step does not fit the batch buffers")
        i = self._next
        self._next = (i + 1) % len(self._hosts)
        if self._events[i] is not None:
            self._events[i].synchronize()
        host = self._hosts[i]
        arr = host.numpy()
        o = self._offsets

        def h(j):
            return arr[o[j]:o[j + 1]]
        h(0)[:T] = token_ids; h(0)[T:pad_tokens] = 0
        h(1)[:T] = positions; h(1)[T:pad_tokens] = 0
        h(2)[:T] = slot_of_token; h(2)[T:pad_tokens] = -1
        h(3)[:B] = seq_slot; h(3)[B:pad_seqs] = -1
        h(4)[:B + 1] = cu_q; h(4)[B + 1:pad_seqs + 1] = cu_q[-1]
        h(5)[:B] = kv_len; h(5)[B:pad_seqs] = 0
        h(6)[:W] = want_rows; h(6)[W:pad_want] = -1
        self.dev.copy_(host, non_blocking=True)
        if self._cuda:
            ev = torch.cuda.Event()
            ev.record()
            self._events[i] = ev

    @property
    def h2d_bytes(self) -> int:
        return self.dev.numel() * 4

    token_ids = property(lambda s: s._d(0))
    positions = property(lambda s: s._d(1))
    slot_of_token = property(lambda s: s._d(2))
    seq_slot = property(lambda s: s._d(3))
    cu_q = property(lambda s: s._d(4))
    kv_len = property(lambda s: s._d(5))
    want_rows = property(lambda s: s._d(6))


@dataclass
class StepBatch:
    """What parts receive.  Counts are the launched (possibly padded) ones."""

    n_tokens: int
    n_seqs: int
    n_want: int
    max_q_len: int
    max_kv_len: int
    is_decode: bool
    token_ids: torch.Tensor
    positions: torch.Tensor
    slot_of_token: torch.Tensor
    seq_slot: torch.Tensor
    cu_q: torch.Tensor
    kv_len: torch.Tensor
    want_rows: torch.Tensor
    host: Optional[HostBatch] = None
    capturing: bool = False
    scratch: dict = field(default_factory=dict)


def pack_entries(slots: Sequence[int], old_lens: Sequence[int], token_lists: Sequence[Sequence[int]],
                 wants: Sequence[Sequence[int]]):
    """Flatten per-sequence token lists into the arrays of a step."""
    for toks, want in zip(token_lists, wants):
        n = len(toks)
        for w in want:
            if not 0 <= w < n:
                raise ValueError(f"wanted place {w} is outside the {n} tokens given")
    if sum(len(t) for t in token_lists) > 256:
        # prompts: whole arrays at a time
        lens = [len(t) for t in token_lists]
        cu_q = np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)
        token_ids = np.concatenate([np.asarray(t, dtype=np.int64) for t in token_lists])
        positions = np.concatenate([np.arange(o, o + n, dtype=np.int64) for o, n in zip(old_lens, lens)])
        slot_of_token = np.repeat(np.asarray(slots, dtype=np.int64), lens)
        kv_len = [o + n for o, n in zip(old_lens, lens)]
        want_rows = [int(cu_q[i]) + w for i, want in enumerate(wants) for w in want]
        return token_ids, positions, slot_of_token, [int(c) for c in cu_q], kv_len, want_rows
    token_ids, positions, slot_of_token, cu_q, kv_len, want_rows = [], [], [], [0], [], []
    for slot, old, toks, want in zip(slots, old_lens, token_lists, wants):
        base = len(token_ids)
        n = len(toks)
        token_ids.extend(int(t) for t in toks)
        positions.extend(range(old, old + n))
        slot_of_token.extend([slot] * n)
        cu_q.append(base + n)
        kv_len.append(old + n)
        want_rows.extend(base + w for w in want)
    return token_ids, positions, slot_of_token, cu_q, kv_len, want_rows
