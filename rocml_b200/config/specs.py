"""Architecture-neutral description of a decoder: what each layer is made of.

An architecture's typed configuration (for example ``Qwen3Config``) is turned
into a ``ModelSpec``.  Everything below the configuration (parts, cache, engine)
reads only these specs, so no part knows which model it sits in, and layers of
one model may differ from one another.

A spec names a *kind* (a string looked up in the part registries of
``rocml_b200.parts``) and carries that kind's sizes and constants.  Kinds that a
test or a user registers later need no change here: ``MixerSpec`` and
``FeedForwardSpec`` keep free-form ``params``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Tuple


def _frozen_params(params: Optional[Mapping[str, Any]]) -> Tuple[Tuple[str, Any], ...]:
    """Parameters as a sorted tuple of pairs; a mapping among the values (``names``) is frozen the same way."""
    return tuple(sorted((k, _frozen_params(v) if isinstance(v, Mapping) else v) for k, v in (params or {}).items()))


def tensor_names(params: Mapping[str, Any], defaults: Mapping[str, str]) -> dict:
    """A part's tensor-name stems: ``defaults`` (role -> stem) overridden by the spec's ``names``
    parameter.  A role the part does not know is an error: it would silently name nothing."""
    given = dict(params.get("names") or ())
    unknown = sorted(set(given) - set(defaults))
    if unknown:
        raise ValueError(f"names for unknown tensors {unknown}; this part has {sorted(defaults)}")
    return {**defaults, **given}


@dataclass(frozen=True)
class NormSpec:
    """A normalisation over the last axis.  kind "rmsnorm": x * rsqrt(mean(x^2) + eps) * w."""

    kind: str = "rmsnorm"
    eps: float = 1e-6


@dataclass(frozen=True)
class PositionSpec:
    """Position encoding applied to queries and keys inside a mixer.

    kind "rope_neox": rotate-half rotary embedding over the first ``rot_dim``
    dimensions of every head with base ``theta``; kind "none": nothing.
    """

    kind: str = "rope_neox"
    theta: float = 1e6
    rot_dim: Optional[int] = None  # None: the whole head
    params_items: Tuple[Tuple[str, Any], ...] = ()

    @property
    def params(self) -> dict:
        return dict(self.params_items)


@dataclass(frozen=True)
class MixerSpec:
    """The token mixer of a layer.  kind "attention" is grouped-query softmax attention.

    Attention params: n_heads, n_kv_heads, head_dim, bias (q/k/v/o biases),
    qk_norm (per-head RMSNorm of q and k before the position encoding),
    qk_norm_eps, window (None: every earlier key; n: the last n keys, the
    query's own position included), scale (None: 1/sqrt(head_dim)),
    names (the tensor-name stems under the layer's mixer prefix, by role:
    q, k, v, o, q_norm, k_norm; default q_proj, k_proj, v_proj, o_proj,
    q_norm, k_norm).
    """

    kind: str
    params_items: Tuple[Tuple[str, Any], ...] = ()
    position: PositionSpec = PositionSpec(kind="none")

    @staticmethod
    def make(kind: str, position: Optional[PositionSpec] = None, **params) -> "MixerSpec":
        return MixerSpec(kind, _frozen_params(params), position or PositionSpec(kind="none"))

    @property
    def params(self) -> dict:
        return dict(self.params_items)


@dataclass(frozen=True)
class FeedForwardSpec:
    """The feed-forward of a layer.  kind "gated_mlp": down(act(gate(x)) * up(x)).

    gated_mlp params: intermediate, activation ("silu"), bias, names (the
    tensor-name stems under the layer's feed-forward prefix, by role: gate,
    up, down; default gate_proj, up_proj, down_proj).
    """

    kind: str
    params_items: Tuple[Tuple[str, Any], ...] = ()

    @staticmethod
    def make(kind: str, **params) -> "FeedForwardSpec":
        return FeedForwardSpec(kind, _frozen_params(params))

    @property
    def params(self) -> dict:
        return dict(self.params_items)


@dataclass(frozen=True)
class LayerSpec:
    """One layer: two norms, a mixer and a feed-forward in a named arrangement.

    arrangement "pre_norm": x += mixer(norm1(x)); x += ff(norm2(x)).
    ``prefix`` is the layer's tensor-name prefix in the weight files; under it the four parts'
    tensors are named ``<prefix>.<mixer_norm_name>.weight``, ``<prefix>.<mixer_name><stem>...``,
    ``<prefix>.<ff_norm_name>.weight`` and ``<prefix>.<ff_name><stem>...`` (the defaults are the
    names of Hugging Face's Qwen3 checkpoints; another architecture gives its own).
    """

    prefix: str
    mixer: MixerSpec
    feed_forward: FeedForwardSpec
    mixer_norm: NormSpec
    ff_norm: NormSpec
    arrangement: str = "pre_norm"
    mixer_norm_name: str = "input_layernorm"
    mixer_name: str = "self_attn."
    ff_norm_name: str = "post_attention_layernorm"
    ff_name: str = "mlp."


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer.  ``layer`` indexes ``ModelSpec.layers``.

    ``reads_cache_of`` names an earlier schedule entry whose cache this run
    reads instead of keeping its own (it then writes nothing).
    """

    layer: int
    reads_cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    """A whole decoder: embedding, layers, the order they run in, final norm, head."""

    architecture: str
    hidden: int
    vocab: int
    max_position: int
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: NormSpec
    tie_embeddings: bool
    embedding_name: str = "model.embed_tokens.weight"
    final_norm_name: str = "model.norm.weight"
    head_name: str = "lm_head.weight"
    stop_tokens: Tuple[int, ...] = ()
    extra: Tuple[Tuple[str, Any], ...] = field(default=())

    def __post_init__(self):
        n = len(self.layers)
        for i, e in enumerate(self.schedule):
            if not 0 <= e.layer < n:
                raise ValueError(f"schedule entry {i} names layer {e.layer}, model has {n}")
            if e.reads_cache_of is not None and not 0 <= e.reads_cache_of < i:
                raise ValueError(
                    f"schedule entry {i} reads the cache of entry {e.reads_cache_of}, "
                    "which must be an earlier entry"
                )
