"""How a layer's parts are arranged."""
from __future__ import annotations

import os
from typing import Dict, List

import torch

from ..config.specs import LayerSpec
from ..profile import scope
from ..weights.decl import TensorDecl
from .base import BuildEnv, ResidualSink, build_feed_forward, build_mixer, build_norm, register_arrangement


# From this many tokens in a step a part is offered to add into the residual itself (the products of
# fewer rows are split over K or run as kernels without that epilogue).
ADD_INTO_MIN_TOKENS = 256


@register_arrangement("pre_norm")
class PreNormBlock:
    """x += mixer(norm1(x)); x += ff(norm2(x)) (rocml/src/forward/mod.rs:281-340).

    The additions are not done here: each part's result travels on as a *delta*, and the
    next norm adds it into the 32-bit residual stream in the same kernel that normalises.
    ``forward`` therefore takes the delta still pending from the layer before and returns
    its own feed-forward's delta."""

    def __init__(self, spec: LayerSpec, hidden: int, env: BuildEnv, mixer_spec=None):
        self.spec = spec
        self.prefix = spec.prefix
        self.mixer_norm = build_norm(spec.mixer_norm, hidden, env)
        self.mixer = build_mixer(mixer_spec or spec.mixer, hidden, env)
        self.ff_norm = build_norm(spec.ff_norm, hidden, env)
        self.ff = build_feed_forward(spec.feed_forward, hidden, env)

    # The four parts' tensor-name prefixes, as the layer's spec gives them.
    def _names(self):
        p, s = self.prefix, self.spec
        return (f"{p}.{s.mixer_norm_name}", f"{p}.{s.mixer_name}", f"{p}.{s.ff_norm_name}", f"{p}.{s.ff_name}")

    def declare(self) -> List[TensorDecl]:
        n1, mx, n2, ff = self._names()
        return self.mixer_norm.declare(n1) + self.mixer.declare(mx) + self.ff_norm.declare(n2) + self.ff.declare(ff)

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        n1, mx, n2, ff = self._names()
        self.mixer_norm.load(tensors, n1)
        self.mixer.load(tensors, mx)
        self.ff_norm.load(tensors, n2)
        self.ff.load(tensors, ff)

    @property
    def graph_safe(self) -> bool:
        return all(p.graph_safe for p in (self.mixer_norm, self.mixer, self.ff_norm, self.ff))

    def weight_bytes(self) -> int:
        return sum(p.weight_bytes() for p in (self.mixer_norm, self.mixer, self.ff_norm, self.ff))

    def workspace_bytes(self, n_tokens: int) -> int:
        """Each half of the layer holds its norm's rows and its part's buffers; the halves follow one another."""
        return max(self.mixer_norm.workspace_bytes(n_tokens) + self.mixer.workspace_bytes(n_tokens),
                   self.ff_norm.workspace_bytes(n_tokens) + self.ff.workspace_bytes(n_tokens))

    def cost(self, q_lens, kv_lens):
        parts = [p.cost(q_lens, kv_lens) for p in (self.mixer_norm, self.mixer, self.ff_norm, self.ff)]
        return sum(p[0] for p in parts), sum(p[1] for p in parts)

    chains = True          # forward() accepts next_block (see below)

    def forward(self, resid, pending, batch, view, next_block=None):
        """``pending`` is what the layer before left: a delta, or a DeferredNorm when it has added its
        result into the residual itself and prepared this layer's first norm.  For a decode step of
        up to 16 tokens the parts are offered to do the same for the norm that follows them
        (ResidualSink), when the part after that norm can take the deferred rows: the norm kernels
        then disappear from the step.  RB_DEFER=0 turns the offers off (and those to prompts, below)."""
        T = batch.n_tokens
        offers = batch.is_decode and T <= 16 and _defer_enabled()     # beyond 16 tokens the norm kernels are cheaper (measured)
        # Prompts: a part may be told to add its result into the residual itself (``add_into``; it then
        # returns None, nothing is pending, and the following norm only normalises): the delta of a
        # few thousand rows then never goes through memory.  Parts that set ``can_add_into`` get the offer.
        adds = not batch.is_decode and T > ADD_INTO_MIN_TOKENS and _defer_enabled()
        with scope(op="mixer_norm"):
            xn = self.mixer_norm.forward(resid, pending, T)
        if offers and getattr(self.mixer, "can_sink", False) and _takes(self.ff, batch):
            delta = self.mixer.forward(xn, batch, view, sink=ResidualSink(resid, self.ff_norm))
        elif adds and getattr(self.mixer, "can_add_into", False):
            delta = self.mixer.forward(xn, batch, view, add_into=resid)
        else:
            delta = self.mixer.forward(xn, batch, view)
        with scope(op="ff_norm"):
            xn = self.ff_norm.forward(resid, delta, T)
        nxt = getattr(next_block, "mixer", None)
        if offers and nxt is not None and getattr(self.ff, "can_sink", False) and _takes(nxt, batch):
            return self.ff.forward(xn, batch, sink=ResidualSink(resid, next_block.mixer_norm))
        if adds and getattr(self.ff, "can_add_into", False):
            return self.ff.forward(xn, batch, add_into=resid)
        return self.ff.forward(xn, batch)


def _takes(part, batch) -> bool:
    f = getattr(part, "takes_deferred", None)
    return bool(f(batch)) if f is not None else False


def _defer_enabled() -> bool:
    return os.environ.get("RB_DEFER", "1") != "0"
