"""The generation loop's decisions, with a scripted executor in place of the engine (no GPU)."""
import pytest

from rocml_b200.engine.generate import GenerateStats, Request, decide, generate, plan_batches
from rocml_b200.errors import RocmlError
from rocml_b200.sampling import SamplingParams


class Scripted:
    """Each sequence emits prompt[0], prompt[0] + 1, ...; records every call."""

    def __init__(self, tokens=1024, slots=8, max_seq_len=64):
        self.max_seq_len = max_seq_len
        self._tokens, self._slots = tokens, slots
        self.free = list(range(slots))
        self.state = {}
        self.calls = []
        self.released = []

    def capacity_tokens(self):
        return self._tokens

    def capacity_slots(self):
        return self._slots

    def new_sequence(self):
        s = self.free.pop(0)
        self.state[s] = None
        return s

    def release(self, slot):
        assert slot in self.state, "released twice"
        del self.state[slot]
        self.released.append(slot)
        self.free.insert(0, slot)

    def run(self, slots, tokens, params, rngs, histories):
        self.calls.append([(s, list(t)) for s, t in zip(slots, tokens)])
        out = []
        for s, t, h in zip(slots, tokens, histories):
            assert s in self.state
            if self.state[s] is None:
                self.state[s] = t[0]
                assert list(h) == list(t)
            else:
                assert len(t) == 1 and h[-1] == t[0]
            self.state[s] += 1
            out.append(self.state[s])
        return out


def test_decide():
    assert decide(7, 0, 5, 10, 64, {7}, False) == (False, "stop")
    assert decide(7, 0, 5, 10, 64, {7}, True) == (True, None)
    assert decide(3, 4, 5, 10, 64, {7}, False) == (True, "length")
    assert decide(3, 0, 5, 65, 64, {7}, False) == (True, "context")
    assert decide(3, 0, 5, 64, 64, {7}, False) == (True, None)


def test_plan_batches_by_count_and_by_pages():
    assert plan_batches([10] * 5, 2, 10_000, 8) == [[0, 1], [2, 3], [4]]
    assert plan_batches([10] * 5, 8, 10_000, 3) == [[0, 1, 2], [3, 4]]
    # 65 tokens take two pages: three such requests fill 6 of 6 pages
    assert plan_batches([65, 65, 65, 1], 8, 6 * 64, 8) == [[0, 1, 2], [3]]
    with pytest.raises(RocmlError):
        plan_batches([1000], 8, 6 * 64, 8)


def test_unequal_prompts_stops_and_early_finish():
    ex = Scripted()
    reqs = [Request([10, 1, 1], 4), Request([20], 2), Request([30, 1], 10, stop_tokens=[33])]
    stats = GenerateStats()
    out = generate(ex, reqs, default_stop=[13], stats=stats)
    assert out[0].tokens == [11, 12] and out[0].finish_reason == "stop"       # 13 is not emitted
    assert out[1].tokens == [21, 22] and out[1].finish_reason == "length"
    assert out[2].tokens == [31, 32] and out[2].finish_reason == "stop"       # its own stop set
    assert [len(c) for c in ex.calls] == [3, 3, 2]                            # the batch shrinks
    assert ex.calls[0][0][1] == [10, 1, 1] and ex.calls[1][0][1] == [11]      # prompts, then one token each
    assert sorted(ex.released) == [0, 1, 2] and not ex.state
    assert stats.prompt_tokens == 6 and stats.batches == 1 and stats.step_batch_sizes == [3, 3, 2]


def test_ignore_eos_and_context_limit_and_callback():
    ex = Scripted(max_seq_len=6)
    out = generate(ex, [Request([10, 0, 0], 100, ignore_eos=True)], default_stop=[11])
    assert out[0].tokens == [11, 12, 13, 14] and out[0].finish_reason == "context"  # 3 + 3 fed = 6 held
    ex = Scripted()
    seen = []
    out = generate(ex, [Request([10], 100)], on_token=lambda i, t: seen.append((i, t)) or t == 12)
    assert out[0].tokens == [11, 12] and out[0].finish_reason == "stop" and seen == [(0, 11), (0, 12)]
    # the callback sees every emitted token, the one that uses up the budget included
    seen = []
    out = generate(Scripted(), [Request([10], 3)], on_token=lambda i, t: seen.append(t) and False)
    assert out[0].tokens == [11, 12, 13] == seen and out[0].finish_reason == "length"


def test_one_batch_after_another_reuses_slots():
    ex = Scripted(slots=2)
    reqs = [Request([100 * i], 2) for i in range(1, 6)]
    out = generate(ex, reqs, max_batch=8)
    assert [c.tokens for c in out] == [[100 * i + 1, 100 * i + 2] for i in range(1, 6)]
    assert len(ex.released) == 5 and set(ex.released) == {0, 1}


def test_zero_budget_and_bad_requests():
    ex = Scripted()
    out = generate(ex, [Request([1], 0), Request([5], 1)])
    assert out[0].tokens == [] and out[0].finish_reason == "length" and out[1].tokens == [6]
    with pytest.raises(RocmlError, match="empty"):
        generate(ex, [Request([], 3)])
    with pytest.raises(RocmlError, match="exceeds"):
        generate(Scripted(max_seq_len=4), [Request([1] * 5, 3)])


def test_each_sequence_gets_its_own_seed():
    class SeedSpy(Scripted):
        def run(self, slots, tokens, params, rngs, histories):
            self.seeds = [r.state for r in rngs]
            return super().run(slots, tokens, params, rngs, histories)
    ex = SeedSpy()
    generate(ex, [Request([1], 1, SamplingParams(0.8, seed=5)), Request([2], 1, SamplingParams(0.8, seed=5))])
    assert ex.seeds == [5, 6]


class Pipelined(Scripted):
    """The same script with launch/collect: the loop may enqueue a step before it has read the
    one before.  Checks what that is allowed to assume."""

    def __init__(self, *a, **kw):
        super().__init__(*a, **kw)
        self.open = []          # handles launched and not yet collected, oldest first
        self.fed = 0

    def launch(self, slots, tokens, params, rngs, histories, feed_from=None):
        if feed_from is None:
            assert not self.open, "host tokens for a step while an earlier step is unread"
            out = Scripted.run(self, slots, tokens, params, rngs, histories)
        else:
            assert self.open and feed_from is self.open[-1], "fed from a step that is not the latest"
            assert list(feed_from["slots"]) == list(slots), "fed step must keep sequences and order"
            assert len(self.open) == 1, "more than one step ahead"
            self.fed += 1
            self.calls.append([(s, ["fed"]) for s in slots])
            out = []
            for s in slots:
                assert s in self.state and self.state[s] is not None
                self.state[s] += 1
                out.append(self.state[s])
        h = {"slots": list(slots), "out": out}
        self.open.append(h)
        return h

    def collect(self, handle):
        assert self.open and handle is self.open[0], "steps are read in the order they were launched"
        self.open.pop(0)
        return handle["out"]


def test_running_ahead_changes_no_result():
    import random
    rnd = random.Random(3)
    for trial in range(40):
        reqs = []
        for _ in range(rnd.randint(1, 7)):
            first = rnd.randint(1, 50) * 100
            stop = first + rnd.randint(1, 12)
            reqs.append(Request([first] + [1] * rnd.randint(0, 5), rnd.randint(0, 9),
                                stop_tokens=[stop] if rnd.random() < 0.6 else None,
                                ignore_eos=rnd.random() < 0.2))
        cb = (lambda i, t: t % 7 == 0) if trial % 3 == 0 else None
        a, b = Scripted(slots=3, max_seq_len=12), Pipelined(slots=3, max_seq_len=12)
        sa, sb = GenerateStats(), GenerateStats()
        out_a = generate(a, reqs, max_batch=3, on_token=cb, stats=sa)
        out_b = generate(b, reqs, max_batch=3, on_token=cb, stats=sb)
        assert [(c.tokens, c.finish_reason) for c in out_a] == [(c.tokens, c.finish_reason) for c in out_b]
        assert not b.state and not b.open and sorted(a.released) == sorted(b.released)
        assert (sa.prompt_tokens, sa.decode_tokens, sa.batches) == (sb.prompt_tokens, sb.decode_tokens, sb.batches)
        out_c = generate(Pipelined(slots=3, max_seq_len=12), reqs, max_batch=3, on_token=cb, run_ahead=False)
        assert [c.tokens for c in out_c] == [c.tokens for c in out_a]


def test_running_ahead_feeds_on_the_device_and_stops_for_a_penalty():
    ex = Pipelined()
    out = generate(ex, [Request([10], 6), Request([20, 1], 6)])
    assert [c.tokens for c in out] == [[11, 12, 13, 14, 15, 16], [21, 22, 23, 24, 25, 26]]
    # prompts from the host, then every further step fed on the device; the last token needs no step
    assert ex.fed == 5 and ex.calls[0][1][1] == [20, 1] and all(t == ["fed"] for c in ex.calls[1:] for _, t in c)
    ex = Pipelined()
    generate(ex, [Request([10], 4, SamplingParams(0.8, repeat_penalty=1.3))])
    assert ex.fed == 0
    # a stop token ends one sequence: the step ahead is read, then the rest goes on from host tokens
    ex = Pipelined()
    out = generate(ex, [Request([10], 6, stop_tokens=[13]), Request([20], 6)])
    assert out[0].tokens == [11, 12] and out[1].tokens == [21, 22, 23, 24, 25, 26]
    assert [len(c) for c in ex.calls] == [2, 2, 2, 2, 1, 1]
    assert ex.calls[4] == [(1, [24])]
