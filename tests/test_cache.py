"""The cache's bookkeeping: no slot or page lost, held twice or freed twice (no GPU)."""
import random

import pytest
import torch

from rocml_b200.cache import FreeList, KVRequirement, SequenceCache, StateRequirement, pages_for
from rocml_b200.errors import CacheError, CacheFull, ContextOverflow


def make(max_tokens=640, max_slots=4, max_seq=512, reqs=None, reads=None, step=None):
    reqs = reqs if reqs is not None else [KVRequirement(2, 16)] * 3
    reads = reads if reads is not None else [None] * len(reqs)
    return SequenceCache(reqs, reads, max_tokens, max_slots, max_seq, torch.float32, "cpu", step)


def test_free_list_refuses_double_free_and_unknown():
    f = FreeList(3, "slot")
    a, b = f.alloc(), f.alloc()
    f.free(a)
    with pytest.raises(CacheError, match="twice"):
        f.free(a)
    with pytest.raises(CacheError):
        f.free(7)
    assert f.alloc() == a  # last freed, first reused
    f.alloc()
    with pytest.raises(CacheFull):
        f.alloc()
    f.check()


def test_groups_by_need():
    reqs = [KVRequirement(2, 16), KVRequirement(2, 16, window=32), KVRequirement(2, 16), StateRequirement((4, 4)), None]
    c = make(reqs=reqs)
    assert len(c.kv_groups) == 2 and len(c.state_groups) == 1
    assert c.views[0].group is c.views[2].group and c.views[0].index == 0 and c.views[2].index == 1
    assert c.views[1].group is not c.views[0].group and c.views[1].group.window == 32
    assert c.views[3].kind == "state" and c.views[4].kind == "none"
    assert tuple(c.views[0].k.shape) == (c.n_pages, 2, 64, 16)


def test_a_layer_can_read_another_layers_cache():
    c = make(reqs=[KVRequirement(2, 16), KVRequirement(2, 16)], reads=[None, 0])
    assert c.views[1].group is c.views[0].group and c.views[1].index == 0 and not c.views[1].writes
    assert c.kv_groups[0].n_entries == 1


def test_growth_pages_and_limits():
    c = make(max_tokens=256, max_slots=3, max_seq=200)
    s = c.alloc_slot()
    assert c.grow(s, 65) == 0
    c.commit(s, 65)
    assert c.length(s) == 65 and c.kv_groups[0].pool.n_held == 2
    c.grow(s, 1); c.commit(s, 1)
    assert c.kv_groups[0].pool.n_held == 2
    with pytest.raises(ContextOverflow):
        c.grow(s, 200)
    t = c.alloc_slot()
    with pytest.raises(CacheFull):
        c.grow(t, 129)  # 3 pages wanted, 2 free
    assert c.kv_groups[0].pool.n_held == 2  # a refused growth takes nothing
    c.grow(t, 128); c.commit(t, 128)
    c.free_slot(s)
    with pytest.raises(CacheError):
        c.free_slot(s)
    with pytest.raises(CacheError):
        c.grow(s, 1)
    c.check_invariants()
    c.free_slot(t)
    assert c.kv_groups[0].pool.n_free == c.n_pages
    c.check_invariants()


def test_window_group_gives_pages_back():
    c = make(max_tokens=1024, max_slots=2, max_seq=1024, reqs=[KVRequirement(1, 16, window=70), KVRequirement(1, 16)])
    win = next(g for g in c.kv_groups if g.window)
    full = next(g for g in c.kv_groups if not g.window)
    s = c.alloc_slot()
    c.grow(s, 300); c.commit(s, 300)
    # the next query sits at 300 and reads keys >= 231: pages 0..2 (keys < 192) are gone
    assert list(win.table_host[s][:5] >= 0) == [False, False, False, True, True]
    assert full.pool.n_held == 5 and win.pool.n_held == 2
    for _ in range(100):
        c.grow(s, 1); c.commit(s, 1)
    assert win.pool.n_held <= 3
    c.check_invariants()
    c.free_slot(s)
    assert win.pool.n_held == 0 and full.pool.n_held == 0


def test_state_is_zero_for_a_new_sequence():
    c = make(reqs=[StateRequirement((3,))])
    s = c.alloc_slot()
    c.views[0].state[s] += 5
    c.free_slot(s)
    assert c.alloc_slot() == s and float(c.views[0].state[s].abs().sum()) == 0


def test_random_traffic_keeps_the_books_straight():
    rng = random.Random(3)
    c = make(max_tokens=64 * 40, max_slots=6, max_seq=64 * 12,
             reqs=[KVRequirement(1, 16), KVRequirement(1, 16, window=100)])
    live = {}
    for _ in range(600):
        op = rng.random()
        if op < 0.25 and c.slots.n_free:
            live[c.alloc_slot()] = 0
        elif op < 0.45 and live:
            s = rng.choice(list(live))
            c.free_slot(s)
            del live[s]
        elif live:
            s = rng.choice(list(live))
            n = rng.choice([1, 1, 1, 17, 64, 130])
            try:
                c.grow(s, n)
                c.commit(s, n)
                live[s] += n
            except (CacheFull, ContextOverflow):
                pass
        c.check_invariants()
        for s, n in live.items():
            assert c.length(s) == n
            assert (c.kv_groups[0].table_host[s] >= 0).sum() == pages_for(n)
    for s in list(live):
        c.free_slot(s)
    c.check_invariants()
    assert all(g.pool.n_held == 0 for g in c.kv_groups) and c.slots.n_held == 0


def _pieces(lens, slots, step):
    """The way the engine cuts a step: sequence after sequence, pieces of at most ``step`` tokens."""
    pieces, cur, room = [], [], step
    for slot, n in zip(slots, lens):
        a = 0
        while a < n:
            take = min(room, n - a)
            cur.append((slot, take))
            a += take
            room -= take
            if room == 0:
                pieces.append(cur)
                cur, room = [], step
    if cur:
        pieces.append(cur)
    return pieces


def test_a_long_prompt_on_a_window_group_goes_in_piece_by_piece():
    """Window 128, pieces of 256 tokens, one slot, a prompt of 3,000 tokens: the window group holds
    pages for a window and a piece only, so the prompt fits piece by piece and not at once."""
    c = make(max_tokens=3072, max_slots=1, max_seq=3072, step=256,
             reqs=[KVRequirement(1, 16, window=128), KVRequirement(1, 16)])
    win = next(g for g in c.kv_groups if g.window)
    assert win.n_pages == pages_for(128 + 256) + 1
    s = c.alloc_slot()
    with pytest.raises(CacheFull):
        c.plan([[(s, 3000)]])
    with pytest.raises(CacheFull):
        c.grow(s, 3000)
    c.check_invariants()
    assert win.pool.n_held == 0
    pieces = _pieces([3000], [s], 256)
    c.plan(pieces)
    peak = 0
    for piece in pieces:
        for slot, n in piece:
            c.grow(slot, n)
        peak = max(peak, win.pool.n_held)
        for slot, n in piece:
            c.commit(slot, n)
        c.check_invariants()
    assert c.length(s) == 3000 and peak <= win.n_pages
    assert win.pool.n_held <= pages_for(128) + 1
    c.free_slot(s)
    c.check_invariants()


def test_plan_agrees_with_what_growth_then_does():
    """plan() says yes exactly when the same pieces, grown and committed one after another, fit;
    and it changes nothing."""
    rng = random.Random(11)
    for trial in range(200):
        step = rng.choice([64, 100, 256])
        window = rng.choice([24, 70, 128, 300])
        max_slots = rng.choice([1, 2, 3])
        c = make(max_tokens=64 * rng.choice([6, 12, 30]), max_slots=max_slots, max_seq=64 * 30, step=step,
                 reqs=[KVRequirement(1, 16, window=window), KVRequirement(1, 16)])
        slots = [c.alloc_slot() for _ in range(max_slots)]
        for s in slots:                          # some history first
            n = rng.choice([0, 1, 63, 64, 200])
            try:
                c.plan([[(s, n)]]) if n else None
                c.grow(s, n); c.commit(s, n)
            except (CacheFull, ContextOverflow):
                pass
        before = [g.pool.n_free for g in c.kv_groups], list(c.lengths)
        lens = [rng.choice([1, 5, 64, 65, 200, 700, 1500]) for _ in slots]
        pieces = _pieces(lens, slots, step)
        try:
            c.plan(pieces)
            ok = True
        except (CacheFull, ContextOverflow):
            ok = False
        assert ([g.pool.n_free for g in c.kv_groups], list(c.lengths)) == before
        try:
            for piece in pieces:
                for slot, n in piece:
                    c.grow(slot, n)
                for slot, n in piece:
                    c.commit(slot, n)
            did = True
        except (CacheFull, ContextOverflow):
            did = False
        assert ok == did, (trial, step, window, lens)
        c.check_invariants()
