"""Interfaces of the parts a layer is put together from, and their registries.

A part is built from its spec (sizes and constants) and a ``BuildEnv`` (device, element
type of activations); it declares the tensors it needs under a name prefix, takes them at
load time, and runs on a ``StepBatch``.  No part knows which model it sits in.

Registering a kind (``register_mixer("name")(cls)`` and the like) is all it takes to make
it usable from a ``ModelSpec``; nothing else in the library names the kinds.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, List, Optional

import torch

from ..cache.requirements import KVRequirement, StateRequirement  # noqa: F401  (re-exported)
from ..config.specs import FeedForwardSpec, MixerSpec, NormSpec, PositionSpec
from ..errors import ConfigError
from ..weights.decl import TensorDecl


@dataclass(frozen=True)
class BuildEnv:
    """Where and how parts compute.  ``act_dtype`` is bfloat16 (serving) or float32 (the true
    32-bit path: no tensor cores, no reduced-precision mode anywhere)."""

    device: torch.device
    act_dtype: torch.dtype

    @property
    def mode(self) -> str:
        return "float32" if self.act_dtype == torch.float32 else "bfloat16"


@dataclass
class ResidualSink:
    """An offer to a part: instead of returning its result as a delta, add it into ``resid`` itself and
    prepare the input of ``norm``, the norm that follows, as a ``DeferredNorm``.  A part may decline by
    returning a delta as always.  Only parts that set ``can_sink`` are made the offer."""

    resid: torch.Tensor       # [T, H] float32
    norm: "Norm"


# A second, simpler offer is made for prompts: ``forward(..., add_into=resid)`` to parts that set
# ``can_add_into``.  The part may add its result into ``resid`` [T, H] float32 itself and return None
# (nothing is pending then), or ignore the offer and return a delta as always.


@dataclass
class DeferredNorm:
    """The output of a norm whose division by the rows' RMS has not happened yet: ``x`` is
    residual * weight in the activations' type (the residual already holds every delta), and column t of
    ``sumsq`` [groups, >= T] float32 sums to row t's sum of squares over ``width`` values.  A part that
    multiplies ``x`` by a matrix applies rsqrt(sum / width + eps) to the product instead.  Only parts
    whose ``takes_deferred(batch)`` says so are handed one."""

    x: torch.Tensor
    sumsq: torch.Tensor
    eps: float
    width: int
    norm: "Norm"
    resid: torch.Tensor

    @property
    def rowscale(self):
        return self.sumsq, self.eps

    def materialize(self) -> torch.Tensor:
        """The rows as the norm itself would have produced them (one more kernel)."""
        return self.norm.forward(self.resid, None, self.x.shape[0], write_back=False)


class Part:
    """Common face: tensors declared, tensors loaded."""

    graph_safe = False  # True when forward() issues only kernels on the current stream

    def declare(self, prefix: str) -> List[TensorDecl]:
        return []

    def load(self, tensors: Dict[str, torch.Tensor], prefix: str) -> None:
        pass

    def weight_bytes(self) -> int:
        """Bytes of weights one forward pass reads (for the roofline)."""
        return 0

    def workspace_bytes(self, n_tokens: int) -> int:
        """Device memory one forward pass over ``n_tokens`` tokens allocates for its intermediate and
        its result (the engine sizes its head room with it)."""
        return 0

    def cost(self, q_lens, kv_lens):
        """(bytes, floating-point operations) one forward pass has to move and do at least, for
        sequences that bring ``q_lens`` tokens and are ``kv_lens`` long afterwards.  The default
        counts the weights once and no arithmetic; parts with products say more."""
        return self.weight_bytes(), 0


class Norm(Part):
    """forward(resid [T, H] float32, delta None | [S, T, H] float32, ...) adds the delta into the
    residual stream in place and returns the normalised rows in the activations' type."""

    def forward(self, resid, delta, n_rows: Optional[int] = None, rows=None, write_back=True):
        raise NotImplementedError


class PositionEncoding(Part):
    """What a mixer needs to place its queries and keys.  ``inv_freq`` (float32 [rot_dim / 2]
    on the device, or None) and ``rot_dim`` drive the fused rotation kernel."""

    inv_freq: Optional[torch.Tensor] = None
    rot_dim: int = 0


class Mixer(Part):
    """forward(xn [T, H], batch, view) -> delta [S, T, H] float32 to be added to the residual.

    ``cache_requirement()`` says what the cache must keep for this layer: a KVRequirement,
    a StateRequirement or None."""

    def cache_requirement(self):
        return None

    def forward(self, xn, batch, view):
        raise NotImplementedError


class FeedForward(Part):
    """forward(xn [T, H], batch) -> delta [S, T, H] float32."""

    def forward(self, xn, batch):
        raise NotImplementedError


_NORMS: Dict[str, Callable] = {}
_POSITIONS: Dict[str, Callable] = {}
_MIXERS: Dict[str, Callable] = {}
_FEED_FORWARDS: Dict[str, Callable] = {}
_ARRANGEMENTS: Dict[str, Callable] = {}


def _register(table, what):
    def outer(kind: str):
        def inner(cls):
            table[kind] = cls
            return cls
        return inner
    return outer


register_norm = _register(_NORMS, "norm")
register_position = _register(_POSITIONS, "position encoding")
register_mixer = _register(_MIXERS, "mixer")
register_feed_forward = _register(_FEED_FORWARDS, "feed-forward")
register_arrangement = _register(_ARRANGEMENTS, "arrangement")


def _lookup(table, kind, what):
    if kind not in table:
        raise ConfigError(f"no {what} of kind {kind!r} is registered (known: {', '.join(sorted(table)) or 'none'})")
    return table[kind]


def build_norm(spec: NormSpec, size: int, env: BuildEnv) -> Norm:
    return _lookup(_NORMS, spec.kind, "norm")(spec, size, env)


def build_position(spec: PositionSpec, head_dim: int, env: BuildEnv) -> PositionEncoding:
    return _lookup(_POSITIONS, spec.kind, "position encoding")(spec, head_dim, env)


def build_mixer(spec: MixerSpec, hidden: int, env: BuildEnv) -> Mixer:
    return _lookup(_MIXERS, spec.kind, "mixer")(spec, hidden, env)


def build_feed_forward(spec: FeedForwardSpec, hidden: int, env: BuildEnv) -> FeedForward:
    return _lookup(_FEED_FORWARDS, spec.kind, "feed-forward")(spec, hidden, env)


def build_block(layer_spec, hidden: int, env: BuildEnv):
    return _lookup(_ARRANGEMENTS, layer_spec.arrangement, "arrangement")(layer_spec, hidden, env)


def registered(kind_of_part: str):
    return tuple(sorted({"norm": _NORMS, "position": _POSITIONS, "mixer": _MIXERS,
                         "feed_forward": _FEED_FORWARDS, "arrangement": _ARRANGEMENTS}[kind_of_part]))
