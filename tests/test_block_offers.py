"""The arrangement's offers to its parts, with toy parts on the CPU (no kernel runs).

A part that feeds the residual stream may be offered a ResidualSink (add your result yourself and
prepare the next norm's rows); it is offered one only when it says it can take it, when the step is a
decode step of few tokens, and when the part after the norm can take the deferred rows.  Parts
without these attributes see the plain interface and nothing else.
"""
import types

import pytest
import torch

from rocml_b200.config.specs import FeedForwardSpec, LayerSpec, MixerSpec, NormSpec
from rocml_b200.parts import (BuildEnv, DeferredNorm, FeedForward, Mixer, Norm, PreNormBlock, ResidualSink,
                              register_feed_forward, register_mixer, register_norm)

LOG = []


@register_norm("toy_norm")
class ToyNorm(Norm):
    deferrable = True

    def __init__(self, spec, size, env):
        self.weight, self.eps = torch.ones(size), spec.eps

    def forward(self, resid, delta, n_rows=None, rows=None, write_back=True):
        if isinstance(delta, DeferredNorm):
            assert delta.norm is self, "a part prepared rows for another norm than the one that follows it"
            LOG.append(("norm passes deferred rows on", id(self)))
            return delta
        if delta is not None:
            resid += delta.sum(0)
        LOG.append(("norm runs", id(self)))
        return resid.clone()


class _Sinks:
    """What a toy part does with an offer: take it (return deferred rows) or not."""

    def finish(self, delta, sink):
        if sink is None:
            return delta
        assert isinstance(sink, ResidualSink)
        sink.resid += delta.sum(0)
        LOG.append((type(self).__name__ + " sinks", id(sink.norm)))
        return DeferredNorm(sink.resid.clone(), torch.ones(1, sink.resid.shape[0]), sink.norm.eps,
                            sink.resid.shape[1], sink.norm, sink.resid)


@register_mixer("toy_plain_mixer")
class PlainMixer(Mixer):
    def __init__(self, spec, hidden, env):
        pass

    def forward(self, xn, batch, view):           # the plain interface: no sink, no deferred rows
        assert isinstance(xn, torch.Tensor)
        return torch.ones((1,) + tuple(xn.shape))


@register_mixer("toy_smart_mixer")
class SmartMixer(Mixer, _Sinks):
    can_sink = True

    def __init__(self, spec, hidden, env):
        pass

    def takes_deferred(self, batch):
        return batch.is_decode

    def forward(self, xn, batch, view, sink=None):
        x = xn.x if isinstance(xn, DeferredNorm) else xn
        return self.finish(torch.ones((1,) + tuple(x.shape)), sink)


@register_feed_forward("toy_plain_ff")
class PlainFF(FeedForward):
    def __init__(self, spec, hidden, env):
        pass

    def forward(self, xn, batch):
        assert isinstance(xn, torch.Tensor)
        return torch.ones((1,) + tuple(xn.shape))


@register_feed_forward("toy_smart_ff")
class SmartFF(FeedForward, _Sinks):
    can_sink = True

    def __init__(self, spec, hidden, env):
        pass

    def takes_deferred(self, batch):
        return True

    def forward(self, xn, batch, sink=None):
        x = xn.x if isinstance(xn, DeferredNorm) else xn
        return self.finish(torch.ones((1,) + tuple(x.shape)), sink)


def block(mixer, ff):
    spec = LayerSpec("l", MixerSpec.make(mixer), FeedForwardSpec.make(ff), NormSpec("toy_norm", 1e-6), NormSpec("toy_norm", 1e-6))
    return PreNormBlock(spec, 4, BuildEnv(torch.device("cpu"), torch.float32))


def batch(tokens, decode):
    return types.SimpleNamespace(n_tokens=tokens, is_decode=decode)


def run(blocks, b):
    LOG.clear()
    resid, pending = torch.zeros(b.n_tokens, 4), None
    for i, blk in enumerate(blocks):
        nxt = blocks[i + 1] if i + 1 < len(blocks) else None
        pending = blk.forward(resid, pending, b, None, next_block=nxt)
    if isinstance(pending, torch.Tensor):
        resid += pending.sum(0)
    return resid, [what for what, _ in LOG]


def test_plain_parts_see_the_plain_interface():
    resid, log = run([block("toy_plain_mixer", "toy_plain_ff")] * 2, batch(3, True))
    assert log == ["norm runs"] * 4 and torch.equal(resid, torch.full((3, 4), 4.0))


def test_offers_are_made_where_they_can_be_taken():
    smart = [block("toy_smart_mixer", "toy_smart_ff") for _ in range(3)]
    resid, log = run(smart, batch(3, True))
    # only the very first norm runs; the last feed-forward has no norm after it and returns a delta
    assert log == ["norm runs", "SmartMixer sinks", "norm passes deferred rows on", "SmartFF sinks",
                   "norm passes deferred rows on", "SmartMixer sinks", "norm passes deferred rows on", "SmartFF sinks",
                   "norm passes deferred rows on", "SmartMixer sinks", "norm passes deferred rows on"]
    assert torch.equal(resid, torch.full((3, 4), 6.0))
    # same sums without the offers: prompts, many tokens, or the switch
    for b in (batch(3, False), batch(17, True)):
        resid, log = run(smart, b)
        assert "SmartMixer sinks" not in log and torch.equal(resid, torch.full((b.n_tokens, 4), 6.0))


def test_no_offer_when_the_next_part_cannot_take_the_rows(monkeypatch):
    mixed = [block("toy_smart_mixer", "toy_plain_ff"), block("toy_plain_mixer", "toy_smart_ff")]
    resid, log = run(mixed, batch(2, True))
    # the smart mixer is followed by a plain feed-forward, the plain mixer cannot sink, and the smart
    # feed-forward of the last block has no norm after it: every norm runs
    assert log == ["norm runs"] * 4 and torch.equal(resid, torch.full((2, 4), 4.0))
    monkeypatch.setenv("RB_DEFER", "0")
    resid, log = run([block("toy_smart_mixer", "toy_smart_ff") for _ in range(2)], batch(2, True))
    assert log == ["norm runs"] * 4


@register_feed_forward("toy_adding_ff")
class AddingFF(FeedForward):
    """Takes the offer made for prompts: adds its result into the residual itself and returns None."""
    can_add_into = True

    def __init__(self, spec, hidden, env):
        pass

    def forward(self, xn, batch, add_into=None):
        delta = torch.ones((1,) + tuple(xn.shape))
        if add_into is None:
            return delta
        add_into += delta.sum(0)
        LOG.append(("AddingFF adds", 0))
        return None


def test_prompts_offer_the_residual_itself(monkeypatch):
    blocks = [block("toy_plain_mixer", "toy_adding_ff") for _ in range(2)]
    resid, log = run(blocks, batch(300, False))          # a prompt of more than 256 tokens
    assert log == ["norm runs", "norm runs", "AddingFF adds", "norm runs", "norm runs", "AddingFF adds"]
    assert torch.equal(resid, torch.full((300, 4), 4.0))
    for b in (batch(300, True), batch(200, False)):     # decode steps and short prompts: no offer
        resid, log = run(blocks, b)
        assert "AddingFF adds" not in log and torch.equal(resid, torch.full((b.n_tokens, 4), 4.0))
    monkeypatch.setenv("RB_DEFER", "0")
    assert "AddingFF adds" not in run(blocks, batch(300, False))[1]
