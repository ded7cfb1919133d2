"""The cache: a slot per sequence, keys and values per layer in pages, per-sequence state.

Layout.  A sequence of the running batch holds a *slot*; its length lives on the host.
Layers are put in *groups* by what they need: every layer that keeps all keys with the
same (kv heads, head size) shares a ``KVGroup``; layers that keep a window of keys form
another group with storage and pages of their own; layers with fixed-size state form
``StateGroup``s.  A KV group stores ``K, V [layers of the group][pages][kv heads][64][head]``
and one block table ``[slots][pages per sequence]`` (page ids, -1 where none), shared by
the group's layers because they grow in step.  Pages of 64 tokens are handed out as a
sequence grows and come back when its slot is freed; a window group also gives back the
pages that fell wholly out of the window.

The reference keeps one sequence: per layer ``K, V [kv heads, max_seq, head]``
(rocml/src/qwen35/cache/mod.rs:86-104), a single ``pos`` (rocml/src/forward/mod.rs:84),
``reset()`` (:229-232), and, for its hybrid family, fixed-size recurrent state beside the
attention planes (rocml/src/qwen35/cache/mod.rs:32-64,180-184).  Here the same pieces are
kept per slot.  Stale contents of reused pages are never read: every kernel is bounded by
the sequence's own length (the argument of rocml/src/forward/mod.rs:224-228).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Union

import numpy as np
import torch

from ..errors import CacheError, CacheFull, ContextOverflow
from .pages import FreeList
from .requirements import KVRequirement, StateRequirement

PAGE = 64


def pages_for(n_tokens: int) -> int:
    return (n_tokens + PAGE - 1) // PAGE


class KVGroup:
    def __init__(self, req: KVRequirement, n_entries: int, n_pages: int, max_slots: int,
                 max_pages_per_seq: int, dtype: torch.dtype, device):
        self.req = req
        self.n_entries = n_entries
        self.n_pages = n_pages
        self.max_pages_per_seq = max_pages_per_seq
        shape = (n_entries, n_pages, req.n_kv_heads, PAGE, req.head_dim)
        self.k = torch.zeros(shape, dtype=dtype, device=device)
        self.v = torch.zeros(shape, dtype=dtype, device=device)
        self.pool = FreeList(n_pages, "page")
        self.table_host = np.full((max_slots, max_pages_per_seq), -1, dtype=np.int32)
        self.table = torch.full((max_slots, max_pages_per_seq), -1, dtype=torch.int32, device=device)
        self._dirty = set()
        self._pins: List[torch.Tensor] = []        # ring of pinned staging copies of the table
        self._pin_events: List[Optional[torch.cuda.Event]] = []
        self._pin_next = 0
        self._released_upto: Dict[int, int] = {}  # slot -> first page a window has not released

    @property
    def window(self) -> Optional[int]:
        return self.req.window

    def bytes(self) -> int:
        return 2 * self.k.numel() * self.k.element_size()

    def ensure(self, slot: int, new_len: int, old_len: int = 0) -> None:
        """Pages for positions < new_len (those a window has released stay released).  ``old_len``: the
        sequence's length so far, whose pages it holds already (only the pages past them are looked at)."""
        need = pages_for(new_len)
        if need > self.max_pages_per_seq:
            raise ContextOverflow(new_len, self.max_pages_per_seq * PAGE)
        row = self.table_host[slot]
        first = max(self._released_upto.get(slot, 0), pages_for(old_len)) if old_len else self._released_upto.get(slot, 0)
        todo = [p for p in range(first, need) if row[p] < 0]
        if len(todo) > self.pool.n_free:
            raise CacheFull(
                f"the cache has {self.pool.n_free} free pages of {PAGE} tokens, {len(todo)} are needed "
                f"(group of {self.n_entries} layers, {self.n_pages} pages in all)"
            )
        for p in todo:
            row[p] = self.pool.alloc()
        if todo:
            self._dirty.add(slot)

    def plan(self, pieces, lengths: Sequence[int]) -> None:
        """The page count of ``ensure`` and ``release_out_of_window`` over a run of pieces (see
        SequenceCache.plan), on numbers only: a sequence holds the pages [first, end) of its row."""
        free = self.pool.n_free
        state: Dict[int, List[int]] = {}
        for n_piece, piece in enumerate(pieces):
            for slot, n_new in piece:
                if slot not in state:
                    # a sequence holds the pages of its length so far, from the first its window has not released
                    state[slot] = [self._released_upto.get(slot, 0), pages_for(lengths[slot]), lengths[slot]]
                st = state[slot]
                st[2] += n_new
                need = pages_for(st[2])
                if need > self.max_pages_per_seq:
                    raise ContextOverflow(st[2], self.max_pages_per_seq * PAGE)
                todo = max(0, need - max(st[0], st[1]))
                if todo > free:
                    raise CacheFull(
                        f"the cache has {free} free pages of {PAGE} tokens when piece {n_piece} of the step "
                        f"starts, {todo} are needed (group of {self.n_entries} layers, {self.n_pages} pages in all"
                        + (f", window of {self.window} tokens" if self.window else "") + ")")
                free -= todo
                st[1] = max(st[1], need)
            if self.window is None:
                continue
            for slot, _ in piece:
                st = state[slot]
                keep_from = max(0, st[2] - self.window + 1) // PAGE
                if keep_from > st[0]:
                    free += max(0, min(keep_from, st[1]) - st[0])
                    st[0] = keep_from

    def release_out_of_window(self, slot: int, length: int) -> None:
        """After a step that left the sequence ``length`` long: the next query sits at a
        position >= length and reads keys >= length - window + 1; pages wholly below go back."""
        if self.window is None:
            return
        keep_from = max(0, length - self.window + 1) // PAGE
        row = self.table_host[slot]
        start = self._released_upto.get(slot, 0)
        for p in range(start, keep_from):
            if row[p] >= 0:
                self.pool.free(int(row[p]))
                row[p] = -1
                self._dirty.add(slot)
        self._released_upto[slot] = max(start, keep_from)

    def release_all(self, slot: int) -> None:
        row = self.table_host[slot]
        for p in np.nonzero(row >= 0)[0]:
            self.pool.free(int(row[p]))
        row[:] = -1
        self._dirty.add(slot)
        self._released_upto.pop(slot, None)

    def flush(self) -> None:
        """Bring the device's block table up to date (before the kernels of a step run)."""
        if not self._dirty:
            return
        if self.table.is_cuda:
            # The copies are asynchronous and the loop above may run a step ahead: each flush stages its
            # rows in the next buffer of a ring and waits for that buffer's previous copies first, so a
            # row that a queued copy still reads is never rewritten (a window group's row may by then
            # name a page that the queued step must not see).
            if not self._pins:
                self._pins = [torch.empty(self.table_host.shape, dtype=torch.int32, pin_memory=True)
                              for _ in range(4)]
                self._pin_events = [None] * len(self._pins)
            i = self._pin_next
            self._pin_next = (i + 1) % len(self._pins)
            if self._pin_events[i] is not None:
                self._pin_events[i].synchronize()
            pin = self._pins[i]
            if len(self._dirty) > 8:
                pin.numpy()[:] = self.table_host
                self.table.copy_(pin, non_blocking=True)
            else:
                for s in sorted(self._dirty):
                    pin.numpy()[s] = self.table_host[s]
                    self.table[s].copy_(pin[s], non_blocking=True)
            ev = torch.cuda.Event()
            ev.record()
            self._pin_events[i] = ev
        else:
            self.table.copy_(torch.from_numpy(self.table_host))
        self._dirty.clear()

    def held_pages(self) -> List[int]:
        return [int(p) for p in self.table_host[self.table_host >= 0]]


class StateGroup:
    def __init__(self, req: StateRequirement, n_entries: int, max_slots: int, device):
        self.req = req
        self.n_entries = n_entries
        self.state = torch.zeros((n_entries, max_slots) + tuple(req.shape), dtype=req.dtype, device=device)

    def bytes(self) -> int:
        return self.state.numel() * self.state.element_size()

    def reset(self, slot: int) -> None:
        self.state[:, slot].zero_()


@dataclass
class CacheView:
    """What one run of a layer sees of the cache."""

    kind: str                      # "kv", "state" or "none"
    group: Union[KVGroup, StateGroup, None] = None
    index: int = 0                 # the layer's place inside its group
    writes: bool = True            # False: it reads another run's cache

    @property
    def k(self):
        return self.group.k[self.index]

    @property
    def v(self):
        return self.group.v[self.index]

    @property
    def block_table(self):
        return self.group.table

    @property
    def state(self):
        return self.group.state[self.index]


Requirement = Union[KVRequirement, StateRequirement, None]


class SequenceCache:
    """Slots, lengths, and the groups' storage.

    ``requirements[i]`` is what schedule entry i needs (None: nothing);
    ``reads_cache_of[i]`` names the entry whose cache entry i reads instead of its own.
    ``max_tokens`` sizes every KV group: the most tokens live sequences hold at once, each
    sequence's count rounded up to a page of 64.
    """

    def __init__(self, requirements: Sequence[Requirement], reads_cache_of: Sequence[Optional[int]],
                 max_tokens: int, max_slots: int, max_seq_len: int, dtype: torch.dtype, device,
                 max_step_tokens: Optional[int] = None):
        if max_tokens <= 0 or max_slots <= 0:
            raise CacheError("the cache needs room for at least one token and one slot")
        self.device = device
        self.dtype = dtype
        self.max_slots = max_slots
        self.n_pages = pages_for(max_tokens)
        self.max_seq_len = min(max_seq_len, self.n_pages * PAGE)
        self.max_pages_per_seq = pages_for(self.max_seq_len)
        self.slots = FreeList(max_slots, "slot")
        self.lengths = [0] * max_slots
        self.kv_groups: List[KVGroup] = []
        self.state_groups: List[StateGroup] = []
        self.views: List[CacheView] = []

        kv_members: Dict[KVRequirement, List[int]] = {}
        st_members: Dict[StateRequirement, List[int]] = {}
        for i, (req, src) in enumerate(zip(requirements, reads_cache_of)):
            if src is not None:
                continue
            if isinstance(req, KVRequirement):
                kv_members.setdefault(req, []).append(i)
            elif isinstance(req, StateRequirement):
                st_members.setdefault(req, []).append(i)
            elif req is not None:
                raise CacheError(f"schedule entry {i} asks for an unknown kind of cache: {req!r}")
        own: Dict[int, CacheView] = {}
        for req, members in kv_members.items():
            n_pages = self.n_pages
            if req.window is not None and max_step_tokens:
                per_seq = pages_for(req.window + max_step_tokens) + 1
                n_pages = min(n_pages, max_slots * per_seq)
            g = KVGroup(req, len(members), n_pages, max_slots, self.max_pages_per_seq, dtype, device)
            self.kv_groups.append(g)
            for j, i in enumerate(members):
                own[i] = CacheView("kv", g, j, True)
        for req, members in st_members.items():
            g = StateGroup(req, len(members), max_slots, device)
            self.state_groups.append(g)
            for j, i in enumerate(members):
                own[i] = CacheView("state", g, j, True)
        for i, (req, src) in enumerate(zip(requirements, reads_cache_of)):
            if src is not None:
                if src not in own:
                    raise CacheError(f"schedule entry {i} reads the cache of entry {src}, which keeps none")
                o = own[src]
                self.views.append(CacheView(o.kind, o.group, o.index, False))
            else:
                self.views.append(own.get(i, CacheView("none")))

    # ---- slots ----------------------------------------------------------------------------
    def alloc_slot(self) -> int:
        s = self.slots.alloc()
        self.lengths[s] = 0
        for g in self.state_groups:
            g.reset(s)
        return s

    def free_slot(self, slot: int) -> None:
        self.slots.free(slot)  # raises on a double free before anything is touched
        for g in self.kv_groups:
            g.release_all(slot)
        self.lengths[slot] = 0

    def length(self, slot: int) -> int:
        self._held(slot)
        return self.lengths[slot]

    def _held(self, slot: int) -> None:
        if not self.slots.is_held(slot):
            raise CacheError(f"slot {slot} is not allocated")

    # ---- growth -----------------------------------------------------------------------------
    def can_hold(self, total_tokens_by_seq: Sequence[int]) -> bool:
        """Would sequences of these final lengths fit an empty cache?"""
        need = sum(pages_for(n) for n in total_tokens_by_seq)
        return need <= self.n_pages and len(total_tokens_by_seq) <= self.max_slots and \
            all(n <= self.max_seq_len for n in total_tokens_by_seq)

    def free_tokens(self) -> int:
        """Room left, in tokens, in the tightest group (whole pages)."""
        if not self.kv_groups:
            return self.n_pages * PAGE
        return min(g.pool.n_free for g in self.kv_groups) * PAGE

    def grow(self, slot: int, n_new: int) -> int:
        """Make room for ``n_new`` more tokens of the slot's sequence; returns its old length.
        Checked before anything launches: ContextOverflow past the longest sequence, CacheFull
        when pages run out."""
        self._held(slot)
        old = self.lengths[slot]
        new = old + n_new
        if new > self.max_seq_len:
            raise ContextOverflow(new, self.max_seq_len)
        for g in self.kv_groups:
            g.ensure(slot, new, old)
        return old

    def plan(self, pieces: Sequence[Sequence[tuple]]) -> None:
        """Would this run of ``grow`` and ``commit`` calls succeed?  ``pieces`` is a list of pieces, each a
        list of (slot, n_new): every sequence of a piece is grown, the piece runs, every sequence is
        committed (a window group then takes back the pages that fell out of the window), and the
        next piece follows.  Nothing is changed; ContextOverflow or CacheFull is raised for the first
        piece that would not fit, so a step that is cut into pieces fails before its first launch
        or not at all."""
        lengths: Dict[int, int] = {}
        for piece in pieces:
            for slot, n_new in piece:
                self._held(slot)
                lengths[slot] = lengths.get(slot, self.lengths[slot]) + n_new
                if lengths[slot] > self.max_seq_len:
                    raise ContextOverflow(lengths[slot], self.max_seq_len)
        for g in self.kv_groups:
            g.plan(pieces, self.lengths)

    def commit(self, slot: int, n_new: int) -> None:
        """The step has been issued: the sequence is n_new longer."""
        self._held(slot)
        self.lengths[slot] += n_new
        for g in self.kv_groups:
            g.release_out_of_window(slot, self.lengths[slot])

    def flush(self) -> None:
        for g in self.kv_groups:
            g.flush()

    # ---- bookkeeping ----------------------------------------------------------------------------
    def bytes(self) -> int:
        return sum(g.bytes() for g in self.kv_groups) + sum(g.bytes() for g in self.state_groups)

    def check_invariants(self) -> None:
        """No slot or page lost, held twice or freed twice."""
        self.slots.check()
        for g in self.kv_groups:
            g.pool.check()
            held = g.held_pages()
            if len(set(held)) != len(held):
                raise CacheError("a page is held by two sequences")
            if len(held) != g.pool.n_held:
                raise CacheError(f"{g.pool.n_held} pages are marked held but the tables name {len(held)}")
            for s in range(self.max_slots):
                if not self.slots.is_held(s) and (g.table_host[s] >= 0).any():
                    raise CacheError(f"free slot {s} still holds pages")
