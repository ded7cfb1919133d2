"""The generation loop: requests in, token lists out.

Requests are served in batches of sequences that start together: the batch's prompts (of
unequal lengths) run in one step, then every live sequence advances by one token per step.
A sequence ends on a stop token (which is not part of its output), at its token budget, or
at the end of the context; its slot goes back at once and the batch carries on with the
rest.  When a batch is finished the next one starts, until every request is served.

While a step runs, the loop may already enqueue the step after it, fed on the device with the
tokens the running step is about to sample: the host reads each step's tokens one step late,
and its own work hides behind the GPU's.  It runs ahead only when every sequence of the step
is sure to go on as far as budget and context decide; a stop token met meanwhile ends its
sequence as always, and the token that was computed ahead for it is dropped.

The decisions (who is batched with whom, when a sequence ends, what the next step holds) are
plain host logic over an ``Executor``; the engine is one executor, a scripted fake in the CPU
tests is another.  The reference's loop does the same for a single sequence: prefill, then
``while !stop && n < max`` with an eos check before the token is emitted and an optional stop
callback (rocml/src/generate/resumed.rs:157-245).
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Callable, Iterable, List, Optional, Protocol, Sequence, Set, Tuple

from ..errors import RocmlError
from ..sampling.params import SamplingParams, XorShift64Star

PAGE = 64


@dataclass
class Request:
    prompt: Sequence[int]
    max_new_tokens: int = 64
    sampling: SamplingParams = SamplingParams()
    stop_tokens: Optional[Iterable[int]] = None   # None: the model's own stop tokens
    ignore_eos: bool = False                      # keep going through stop tokens (benchmarks)


@dataclass
class Completion:
    tokens: List[int]
    finish_reason: str        # "stop", "length" (token budget) or "context" (no room left)
    prompt_tokens: int


@dataclass
class GenerateStats:
    """Counts and times of one generate call (rocml/src/generate/mod.rs:26-59)."""

    prompt_tokens: int = 0
    decode_tokens: int = 0
    prefill_seconds: float = 0.0
    decode_seconds: float = 0.0
    batches: int = 0
    step_batch_sizes: List[int] = field(default_factory=list)

    @property
    def prompt_tokens_per_sec(self) -> float:
        return self.prompt_tokens / self.prefill_seconds if self.prefill_seconds > 0 else 0.0

    @property
    def decode_tokens_per_sec(self) -> float:
        return self.decode_tokens / self.decode_seconds if self.decode_seconds > 0 else 0.0


class Executor(Protocol):
    """What the loop needs from an engine.  ``launch`` and ``collect`` are optional: an executor
    that has them lets the loop run one step ahead."""

    max_seq_len: int

    def capacity_tokens(self) -> int: ...
    def capacity_slots(self) -> int: ...
    def new_sequence(self) -> int: ...
    def release(self, slot: int) -> None: ...
    def run(self, slots: Sequence[int], tokens: Sequence[Sequence[int]], params: Sequence[SamplingParams],
            rngs: Sequence[XorShift64Star], histories: Sequence[Sequence[int]]) -> List[int]:
        """Step the given sequences with the given next tokens and sample one token each."""

    # def launch(self, slots, tokens, params, rngs, histories, feed_from=None) -> handle
    #     the same, enqueued only; with feed_from (the handle of the step before, same sequences,
    #     same order) the next tokens are that step's samples and ``tokens`` is not read
    # def collect(self, handle) -> List[int]


class _Sync:
    """launch/collect over an executor that only has ``run``: the step runs when it is collected, so
    that the loop's clock, which brackets ``collect``, sees it."""

    def __init__(self, executor):
        self.run = executor.run

    def launch(self, slots, tokens, params, rngs, histories, feed_from=None):
        return (list(slots), [list(t) for t in tokens], list(params), list(rngs), [h for h in histories])

    def collect(self, handle):
        return self.run(*handle)


def _pages(n: int) -> int:
    return (n + PAGE - 1) // PAGE


def plan_batches(needs: Sequence[int], max_batch: int, capacity_tokens: int, capacity_slots: int) -> List[List[int]]:
    """Cut the requests, in order, into batches.  ``needs[i]`` is the most tokens request i can
    come to hold (prompt + new tokens); a batch takes requests while it stays within
    ``max_batch`` sequences, the slots, and the cache's pages of 64 tokens."""
    limit = max(1, min(max_batch, capacity_slots))
    cap_pages = capacity_tokens // PAGE
    batches, cur, used = [], [], 0
    for i, n in enumerate(needs):
        p = _pages(n)
        if p > cap_pages:
            raise RocmlError(
                f"request {i} can come to hold {n} tokens; the cache holds {cap_pages * PAGE}")
        if cur and (len(cur) >= limit or used + p > cap_pages):
            batches.append(cur)
            cur, used = [], 0
        cur.append(i)
        used += p
    if cur:
        batches.append(cur)
    return batches


def decide(token: int, n_generated: int, max_new_tokens: int, length_after: int, max_seq_len: int,
           stop_tokens: Set[int], ignore_eos: bool) -> Tuple[bool, Optional[str]]:
    """What to do with a freshly sampled token: (emit it?, finish reason or None).

    ``n_generated`` counts tokens emitted before this one; ``length_after`` is the sequence's
    length in the cache if this token is fed back.  A stop token ends the sequence and is not
    emitted (rocml/src/generate/resumed.rs:217-219); the budget ends it after the token is
    emitted; so does a context with no room for the next token."""
    if not ignore_eos and token in stop_tokens:
        return False, "stop"
    if n_generated + 1 >= max_new_tokens:
        return True, "length"
    if length_after > max_seq_len:
        return True, "context"
    return True, None


def generate(executor: Executor, requests: Sequence[Request], default_stop: Iterable[int] = (),
             max_batch: int = 64, on_token: Optional[Callable[[int, int], bool]] = None,
             stats: Optional[GenerateStats] = None, run_ahead: bool = True) -> List[Completion]:
    """Serve every request; ``on_token(request index, token)`` may return True to end that
    sequence after the token (the reference's stop callback, resumed.rs:220-230).  With
    ``run_ahead`` off every step is read before the next is enqueued; the tokens are the same."""
    stats = stats if stats is not None else GenerateStats()
    default_stop = set(default_stop)
    limit = executor.max_seq_len
    needs = []
    for i, r in enumerate(requests):
        if len(r.prompt) == 0:
            raise RocmlError(f"request {i} has an empty prompt")
        if len(r.prompt) > limit:
            raise RocmlError(f"request {i}: prompt of {len(r.prompt)} tokens exceeds the context of {limit}")
        needs.append(min(len(r.prompt) + max(r.max_new_tokens, 0), limit))
    results: List[Optional[Completion]] = [None] * len(requests)
    pipelined = run_ahead and hasattr(executor, "launch") and hasattr(executor, "collect")
    ex = executor if pipelined else _Sync(executor)
    for batch in plan_batches(needs, max_batch, executor.capacity_tokens(), executor.capacity_slots()):
        stats.batches += 1
        live = []
        for j, i in enumerate(batch):
            r = requests[i]
            if r.max_new_tokens <= 0:
                results[i] = Completion([], "length", len(r.prompt))
                continue
            stops = default_stop if r.stop_tokens is None else set(r.stop_tokens)
            live.append({"i": i, "req": r, "slot": executor.new_sequence(), "out": [], "done": False,
                         "history": list(r.prompt), "stops": stops,
                         "rng": XorShift64Star(r.sampling.seed + j), "next": list(r.prompt)})
        if not live:
            continue

        def launch(seqs, feed_from=None):
            return ex.launch([s["slot"] for s in seqs], [s["next"] for s in seqs],
                             [s["req"].sampling for s in seqs], [s["rng"] for s in seqs],
                             [s["history"] for s in seqs], feed_from=feed_from)

        t_batch = time.perf_counter()
        flying, handle = live, launch(live)      # the step whose tokens are read next
        first = True
        while flying:
            t0 = t_batch if first else time.perf_counter()     # the prompts' time includes their launch
            ahead = None
            if pipelined and all(_goes_on_for_sure(s, limit) for s in flying):
                ahead = launch(flying, feed_from=handle)
            tokens = ex.collect(handle)
            still = []
            n_read = 0
            for s, tok in zip(flying, tokens):
                if s["done"]:
                    continue                      # it ended while this step was already on its way
                n_read += 1
                r = s["req"]
                length_after = len(s["history"]) + 1
                emit, reason = decide(tok, len(s["out"]), r.max_new_tokens, length_after, limit,
                                      s["stops"], r.ignore_eos)
                if emit:
                    s["out"].append(tok)
                    s["history"].append(tok)
                    if on_token is not None and on_token(s["i"], tok) and reason is None:
                        reason = "stop"       # the callback sees every emitted token; its answer ends a sequence that would go on
                if reason is None:
                    s["next"] = [tok]
                    still.append(s)
                else:
                    s["done"] = True
                    executor.release(s["slot"])
                    results[s["i"]] = Completion(s["out"], reason, len(r.prompt))
            if ahead is not None and not still:
                ex.collect(ahead)                 # everyone ended: nothing of that step is kept
                ahead = None
            dt = time.perf_counter() - t0
            stats.step_batch_sizes.append(n_read)
            if first:
                stats.prefill_seconds += dt
                stats.prompt_tokens += sum(len(requests[s["i"]].prompt) for s in flying)
                first = False
            else:
                stats.decode_seconds += dt
                stats.decode_tokens += n_read
            if ahead is not None:
                handle = ahead                    # same rows; ended ones are skipped when it is read
            elif still:
                flying, handle = still, launch(still)
            else:
                flying = []
    return results


def _goes_on_for_sure(s, limit: int) -> bool:
    """Whether the sequence takes another step after the token now being sampled, as far as
    budget and context decide (a stop token can still end it).  Sequences with a repeat penalty
    never run ahead: the penalty reads the history on the host, which is one token behind."""
    if s["done"] or s["req"].sampling.repeat_penalty is not None:
        return False
    return len(s["out"]) + 1 < s["req"].max_new_tokens and len(s["history"]) + 1 <= limit
