"""A plain restatement of the reference's host sampler (rocml/src/sample.rs), for tests.

Order of operations (sample.rs:90-166): repeat penalty over the last ``window`` history
ids (divide a positive logit, multiply a non-positive one: :188-202) -> temperature <= 0
means argmax, first maximum wins (:172-182) -> multiply by 1/temperature (:102-105) ->
keep the top_k largest, k clamped to [1, V] (:110-116) -> softmax over the survivors with
the maximum subtracted (:118-131) -> top_p clamped to [0, 1]: sort descending, keep the
shortest prefix whose cumulative probability reaches top_p, at least one (:138-153) ->
threshold = u * total; walk the survivors (sorted order if top_p was applied, else index
order) until the cumulative sum reaches it (:155-165).  RNG: xorshift64* (:69-76), seed 0
remapped (:61-67), u = (next >> 40) / 2^24 (:80-82).

One deliberate difference: without top_p the reference multiplies u by the sum of the
UNNORMALISED exponentials (sample.rs:133,143 keep ``sum`` as ``effective_total``) while it
walks normalised probabilities, so most draws overshoot and fall back to the first
candidate.  Here, as in the library, the threshold is u times the sum of the probabilities
actually walked, which is what the surrounding code and its tests intend.
"""
import numpy as np

MASK = (1 << 64) - 1


class XorShift64Star:
    def __init__(self, seed):
        self.s = 0x9E3779B97F4A7C15 if seed == 0 else (seed & MASK)

    def next_u64(self):
        x = self.s
        x ^= x >> 12
        x ^= (x << 25) & MASK
        x ^= x >> 27
        self.s = x
        return (x * 0x2545F4914F6CDD1D) & MASK

    def next_f32(self):
        return np.float32(self.next_u64() >> 40) / np.float32(1 << 24)


def sample(logits, history, temperature=0.0, top_k=None, top_p=None, rng=None,
           repeat_penalty=None, window=64):
    scored = np.array(logits, dtype=np.float32).copy()
    if repeat_penalty is not None and repeat_penalty > 0 and abs(repeat_penalty - 1.0) >= np.finfo(np.float32).eps:
        for t in history[max(0, len(history) - window):]:
            if 0 <= t < len(scored):
                scored[t] = scored[t] / np.float32(repeat_penalty) if scored[t] > 0 else scored[t] * np.float32(repeat_penalty)
    if temperature <= 0:
        return int(np.argmax(scored))  # numpy's argmax returns the first maximum
    scored *= np.float32(1.0) / np.float32(temperature)
    idx = np.arange(len(scored))
    if top_k is not None:
        k = min(max(int(top_k), 1), len(scored))
        idx = np.argsort(-scored, kind="stable")[:k]
        idx = np.sort(idx)  # unsorted candidate set; index order is what the walk uses without top_p
    probs = np.exp(scored[idx] - scored[idx].max()).astype(np.float32)
    total = np.float32(probs.sum(dtype=np.float32))
    if total > 0:
        probs = probs / total
    order = np.arange(len(idx))
    eff = np.float32(probs.sum(dtype=np.float32))
    if top_p is not None:
        p = min(max(float(top_p), 0.0), 1.0)
        order = np.argsort(-probs, kind="stable")
        cum = np.cumsum(probs[order], dtype=np.float32)
        hit = np.nonzero(cum >= np.float32(p))[0]
        cutoff = max(int(hit[0]) + 1 if len(hit) else len(order), 1)
        order = order[:cutoff]
        eff = np.float32(probs[order].sum(dtype=np.float32))
    thr = rng.next_f32() * max(eff, np.finfo(np.float32).tiny)
    acc = np.float32(0)
    for i in order:
        acc += probs[i]
        if acc >= thr:
            return int(idx[i])
    return int(idx[order[0]])
