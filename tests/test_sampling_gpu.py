"""The GPU sampler against the plain sampler (tests/plain_sampler.py) and against float64 arithmetic."""
import numpy as np
import pytest
import torch

from plain_sampler import XorShift64Star as PlainRng, sample as plain_sample

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def make_logits(seed, V, scale=3.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(V, generator=g) * scale).float()


def gpu_draws(logits, n, history=(), **kw):
    """n successive draws of one sequence with the library's sampler (fresh logits every time)."""
    from rocml_b200.sampling import Sampler, SamplingParams, XorShift64Star
    sp = SamplingParams(**kw)
    s = Sampler(DEV, max_batch=4)
    rng = XorShift64Star(sp.seed)
    out = []
    for _ in range(n):
        out.append(s.sample(logits.to(DEV)[None, :].clone(), [sp], [rng], [list(history)])[0])
    return out


@pytest.mark.parametrize("V", [311, 5000, 151936])
def test_greedy_is_the_first_maximum(V):
    from rocml_b200.sampling import Sampler, SamplingParams
    logits = make_logits(1, V)
    logits[V // 2] = logits[V - 3] = logits.max() + 1.0   # a tie: the first index wins
    s = Sampler(DEV, max_batch=4)
    batch = torch.stack([logits, make_logits(2, V)]).to(DEV)
    got = s.sample(batch, [SamplingParams()] * 2, [None, None], [[], []])
    assert got == [V // 2, int(torch.argmax(make_logits(2, V)))]


@pytest.mark.parametrize("V", [311, 5000, 151936])
@pytest.mark.parametrize("kw", [dict(temperature=0.6, top_k=20, top_p=0.95), dict(temperature=1.0, top_k=50),
                                dict(temperature=0.8, top_k=1), dict(temperature=1.3, top_k=700, top_p=0.5)])
def test_top_k_route_equals_the_plain_sampler(V, kw):
    logits = make_logits(3, V)
    for seed in (0, 7):
        got = gpu_draws(logits, 40, seed=seed, **kw)
        rng = PlainRng(seed)
        want = [plain_sample(logits.numpy(), [], rng=rng, **kw) for _ in range(40)]
        assert got == want


def exact_reference(logits, u, temperature, top_k=None, top_p=None):
    """The same procedure in float64 (the order of the sums then does not matter)."""
    s = logits.double().numpy() * np.float64(np.float32(1.0) / np.float32(temperature))
    s = (logits.numpy() * (np.float32(1.0) / np.float32(temperature))).astype(np.float64)
    keep = np.ones(len(s), bool)
    if top_k is not None and top_k < len(s):
        kth = np.sort(s)[-top_k]
        keep = s >= kth
    p = np.where(keep, np.exp(s - s.max()), 0.0)
    if top_p is not None:
        order = np.argsort(-s, kind="stable")
        order = order[keep[order]]
        cum = np.cumsum(p[order])
        cut = int(np.nonzero(cum >= top_p * cum[-1])[0][0]) + 1
        order = order[:cut]
    else:
        order = np.nonzero(keep)[0]
    cum = np.cumsum(p[order])
    thr = max(u * cum[-1], 1e-300)
    return int(order[np.nonzero(cum >= thr)[0][0]])


@pytest.mark.parametrize("V", [311, 20011])
@pytest.mark.parametrize("kw", [dict(temperature=1.0), dict(temperature=0.7, top_p=0.9),
                                dict(temperature=1.5, top_k=3000), dict(temperature=1.0, top_k=3000, top_p=0.8)])
def test_whole_row_route_equals_float64(V, kw):
    from rocml_b200.sampling import XorShift64Star
    logits = make_logits(5, V, scale=2.0)
    got = gpu_draws(logits, 60, seed=11, **kw)
    rng = XorShift64Star(11)
    want = [exact_reference(logits, rng.next_f32(), **kw) for _ in range(60)]
    assert got == want


def test_frequencies_follow_the_softmax():
    logits = torch.tensor([2.0, 1.0, 0.0, -1.0, 0.5, 1.5, -3.0])
    draws = gpu_draws(logits, 3000, temperature=1.0, seed=3)
    freq = np.bincount(draws, minlength=7) / 3000.0
    want = torch.softmax(logits, 0).numpy()
    assert np.abs(freq - want).max() < 0.03


def test_repeat_penalty():
    from rocml_b200.sampling import Sampler, SamplingParams
    logits = torch.tensor([0.1, 2.0, -1.0, 2.0, 0.5])
    s = Sampler(DEV, max_batch=2)
    sp = SamplingParams(repeat_penalty=10.0, repeat_penalty_window=2)
    assert s.sample(logits[None].to(DEV).clone(), [sp], [None], [[1, 3]])[0] == 4
    assert s.sample(logits[None].to(DEV).clone(), [sp], [None], [[1, 3, 0]])[0] == 1   # the window forgot id 1
    rng_kw = dict(temperature=0.5, top_k=3, repeat_penalty=1.3)
    want = plain_sample(logits.numpy(), [3, 3, 1], rng=PlainRng(2), window=64, **rng_kw)
    got = gpu_draws(logits, 1, seed=2, history=[3, 3, 1], **{k: v for k, v in rng_kw.items()})
    assert got == [want]


@pytest.mark.parametrize("kw", [dict(temperature=1.0), dict(temperature=0.7, top_p=0.9),
                                dict(temperature=1.5, top_k=3000), dict(temperature=1.0, top_k=3000, top_p=0.8),
                                dict(temperature=0.9, top_k=40, top_p=0.7)])
def test_wide_rows_with_ties_and_masked_stretches(kw):
    """A row wide enough to be cut over several blocks, whose values repeat thousands of times (so that
    thresholds fall inside runs of equal values, which enter in index order, and a bin holds more
    elements than fit in shared memory) and of which a stretch across two parts is masked out."""
    from rocml_b200.sampling import XorShift64Star
    V = 40004
    logits = (make_logits(9, V, scale=2.0) * 4).round() / 4
    logits[4900:10300] = -float("inf")
    got = gpu_draws(logits, 60, seed=5, **kw)
    rng = XorShift64Star(5)
    want = [exact_reference(logits, rng.next_f32(), **kw) for _ in range(60)]
    assert got == want


def test_rows_of_a_batch_sample_each_in_its_own_way():
    """Wide rows of one launch with different parameters, a penalty among them, in a matrix whose rows
    do not start on 16-byte boundaries: every row equals the same row sampled alone."""
    from rocml_b200.sampling import Sampler, SamplingParams, XorShift64Star
    V = 30001
    ways = [SamplingParams(), SamplingParams(0.8, top_k=30, top_p=0.9, seed=1), SamplingParams(1.1, seed=2),
            SamplingParams(0.7, top_p=0.8, seed=3, repeat_penalty=1.5, repeat_penalty_window=8),
            SamplingParams(repeat_penalty=50.0), SamplingParams(1.0, top_k=2000, seed=4)]
    rows = [make_logits(20 + i, V, scale=2.0) for i in range(len(ways))]
    top = int(rows[4].argmax())
    histories = [[], [], [], [int(rows[3].argmax()), 5, 6], [top], []]
    alone = []
    for sp, row, h in zip(ways, rows, histories):
        s = Sampler(DEV, max_batch=8)
        rng = XorShift64Star(sp.seed)
        alone.append([s.sample(row.to(DEV)[None].clone(), [sp], [rng], [h])[0] for _ in range(5)])
    assert alone[4][0] != top                                        # the penalty moved the maximum
    s = Sampler(DEV, max_batch=8)
    rngs = [XorShift64Star(sp.seed) for sp in ways]
    together = []
    for _ in range(5):
        together.append(s.sample(torch.stack(rows).to(DEV), ways, rngs, histories))
    assert [list(col) for col in zip(*together)] == alone
