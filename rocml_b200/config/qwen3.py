"""Typed configuration of the dense Qwen3 decoder, read from config.json.

Field-for-field this is the reference's ``ModelConfig``
(rocml/src/config.rs:31-54) with the Hugging Face key names in place of the
GGUF ones, and the same checks (rocml/src/config.rs:84-114): non-zero sizes,
query heads a multiple of key/value heads, an even head size.  Keys the
reference never reads but Qwen3 checkpoints carry (attention_bias, the
sliding-window keys, tie_word_embeddings) are honoured rather than ignored;
rope scaling is rejected because no formula for it exists in the reference.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, asdict
from typing import Any, Mapping, Optional, Tuple

from ..errors import ConfigError, ModelFileMissing
from .specs import (
    FeedForwardSpec,
    LayerSpec,
    MixerSpec,
    ModelSpec,
    NormSpec,
    PositionSpec,
    ScheduleEntry,
)

ARCHITECTURE = "Qwen3ForCausalLM"

_FULL = "full_attention"
_SLIDING = "sliding_attention"


def _as_int(d: Mapping[str, Any], key: str, default=None) -> int:
    v = d.get(key, default)
    if v is None:
        raise ConfigError(f"config.json lacks {key!r}")
    if isinstance(v, bool) or not isinstance(v, int):
        raise ConfigError(f"config.json: {key!r} must be an integer, found {v!r}")
    return v


def _as_float(d: Mapping[str, Any], key: str, default=None) -> float:
    v = d.get(key, default)
    if v is None:
        raise ConfigError(f"config.json lacks {key!r}")
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json: {key!r} must be a number, found {v!r}")
    return float(v)


def _token_ids(v) -> Tuple[int, ...]:
    if v is None:
        return ()
    if isinstance(v, int) and not isinstance(v, bool):
        return (v,)
    if isinstance(v, (list, tuple)) and all(isinstance(t, int) for t in v):
        return tuple(v)
    raise ConfigError(f"config.json: eos_token_id must be an integer or a list, found {v!r}")


@dataclass(frozen=True)
class Qwen3Config:
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    vocab_size: int
    max_position_embeddings: int
    rope_theta: float
    rms_norm_eps: float
    tie_word_embeddings: bool = False
    attention_bias: bool = False
    hidden_act: str = "silu"
    # One entry per layer: None for full attention, else the window in tokens.
    layer_windows: Tuple[Optional[int], ...] = ()
    eos_token_ids: Tuple[int, ...] = ()
    bos_token_id: Optional[int] = None
    torch_dtype: str = "bfloat16"

    # ---- derived sizes (rocml/src/config.rs:134-144) -------------------------
    @property
    def q_dim(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def kv_group_size(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads

    # ---- construction --------------------------------------------------------
    def __post_init__(self):
        self.validate()

    def validate(self) -> None:
        for key in ("hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                    "num_key_value_heads", "head_dim", "vocab_size", "max_position_embeddings"):
            if getattr(self, key) <= 0:
                raise ConfigError(f"{key} must be positive, found {getattr(self, key)}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(
                f"num_attention_heads {self.num_attention_heads} is not a multiple of "
                f"num_key_value_heads {self.num_key_value_heads} (needed to map query heads to "
                "key/value heads)"
            )
        if self.head_dim % 2:
            raise ConfigError(f"head_dim {self.head_dim} must be even (rotary pairs)")
        if not self.rope_theta > 0:
            raise ConfigError(f"rope_theta must be positive, found {self.rope_theta}")
        if not self.rms_norm_eps > 0:
            raise ConfigError(f"rms_norm_eps must be positive, found {self.rms_norm_eps}")
        if self.hidden_act != "silu":
            raise ConfigError(f"hidden_act {self.hidden_act!r} is not supported (only 'silu')")
        if self.layer_windows and len(self.layer_windows) != self.num_hidden_layers:
            raise ConfigError(
                f"{len(self.layer_windows)} layer windows for {self.num_hidden_layers} layers"
            )
        for w in self.layer_windows:
            if w is not None and w <= 0:
                raise ConfigError(f"sliding_window must be positive, found {w}")

    @staticmethod
    def from_dict(d: Mapping[str, Any]) -> "Qwen3Config":
        archs = d.get("architectures") or []
        if archs and archs[0] != ARCHITECTURE:
            raise ConfigError(f"architectures[0] is {archs[0]!r}, expected {ARCHITECTURE!r}")
        hidden = _as_int(d, "hidden_size")
        heads = _as_int(d, "num_attention_heads")
        layers = _as_int(d, "num_hidden_layers")
        if heads <= 0:
            raise ConfigError(f"num_attention_heads must be positive, found {heads}")
        head_dim = d.get("head_dim")
        if head_dim is None:
            if hidden % heads:
                raise ConfigError(
                    f"head_dim is absent and hidden_size {hidden} is not a multiple of "
                    f"num_attention_heads {heads}"
                )
            head_dim = hidden // heads
        elif isinstance(head_dim, bool) or not isinstance(head_dim, int):
            raise ConfigError(f"config.json: 'head_dim' must be an integer, found {head_dim!r}")

        rope = d.get("rope_parameters") or {}
        theta = d.get("rope_theta", rope.get("rope_theta"))
        if theta is None:
            raise ConfigError("config.json lacks 'rope_theta'")
        scaling = d.get("rope_scaling")
        if scaling is None and rope.get("rope_type", "default") != "default":
            scaling = rope
        if scaling is not None:
            kind = scaling.get("rope_type", scaling.get("type", "default")) if isinstance(scaling, Mapping) else scaling
            if kind != "default":
                raise ConfigError(f"rope_scaling {scaling!r} is not supported (plain rotary only)")

        windows: Tuple[Optional[int], ...] = ()
        layer_types = d.get("layer_types")
        use_sliding = bool(d.get("use_sliding_window", False))
        if layer_types is not None:
            if len(layer_types) != layers:
                raise ConfigError(f"layer_types has {len(layer_types)} entries for {layers} layers")
            bad = sorted({t for t in layer_types if t not in (_FULL, _SLIDING)})
            if bad:
                raise ConfigError(f"layer_types holds unknown kinds {bad}")
            if _SLIDING in layer_types:
                win = _as_int(d, "sliding_window")
                windows = tuple(win if t == _SLIDING else None for t in layer_types)
        elif use_sliding:
            win = _as_int(d, "sliding_window")
            first = _as_int(d, "max_window_layers")
            windows = tuple(win if i >= first else None for i in range(layers))
        if windows and all(w is None for w in windows):
            windows = ()

        return Qwen3Config(
            hidden_size=hidden,
            intermediate_size=_as_int(d, "intermediate_size"),
            num_hidden_layers=layers,
            num_attention_heads=heads,
            num_key_value_heads=_as_int(d, "num_key_value_heads", heads),
            head_dim=head_dim,
            vocab_size=_as_int(d, "vocab_size"),
            max_position_embeddings=_as_int(d, "max_position_embeddings"),
            rope_theta=float(theta),
            rms_norm_eps=_as_float(d, "rms_norm_eps"),
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            attention_bias=bool(d.get("attention_bias", False)),
            hidden_act=str(d.get("hidden_act", "silu")),
            layer_windows=windows,
            eos_token_ids=_token_ids(d.get("eos_token_id")),
            bos_token_id=d.get("bos_token_id"),
            torch_dtype=str(d.get("torch_dtype", d.get("dtype", "bfloat16"))),
        )

    @staticmethod
    def from_json(path: str) -> "Qwen3Config":
        if os.path.isdir(path):
            path = os.path.join(path, "config.json")
        if not os.path.isfile(path):
            raise ModelFileMissing(f"no config.json at {path}")
        try:
            with open(path, "r", encoding="utf-8") as f:
                d = json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path} is not valid JSON: {e}") from e
        if not isinstance(d, dict):
            raise ConfigError(f"{path} does not hold a JSON object")
        return Qwen3Config.from_dict(d)

    def to_dict(self) -> dict:
        """The config.json this configuration is read back from."""
        d = {
            "architectures": [ARCHITECTURE],
            "model_type": "qwen3",
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "vocab_size": self.vocab_size,
            "max_position_embeddings": self.max_position_embeddings,
            "rope_theta": self.rope_theta,
            "rope_scaling": None,
            "rms_norm_eps": self.rms_norm_eps,
            "tie_word_embeddings": self.tie_word_embeddings,
            "attention_bias": self.attention_bias,
            "hidden_act": self.hidden_act,
            "torch_dtype": self.torch_dtype,
        }
        if self.layer_windows:
            d["use_sliding_window"] = True
            d["sliding_window"] = next(w for w in self.layer_windows if w is not None)
            d["layer_types"] = [_SLIDING if w is not None else _FULL for w in self.layer_windows]
        else:
            d["use_sliding_window"] = False
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids) if len(self.eos_token_ids) > 1 else self.eos_token_ids[0]
        if self.bos_token_id is not None:
            d["bos_token_id"] = self.bos_token_id
        return d

    # ---- the architecture, spelled as parts ------------------------------------
    def to_model_spec(self) -> ModelSpec:
        """Embedding; N pre-norm layers of (GQA attention with per-head q/k RMSNorm and
        rotate-half rotary, SwiGLU MLP); final RMSNorm; tied or untied head
        (rocml/src/forward/mod.rs:271-378, attention.rs:30-249, ffn.rs:17-112)."""
        norm = NormSpec("rmsnorm", self.rms_norm_eps)
        pos = PositionSpec("rope_neox", theta=self.rope_theta, rot_dim=None)
        ff = FeedForwardSpec.make(
            "gated_mlp", intermediate=self.intermediate_size, activation=self.hidden_act, bias=False
        )
        layers = []
        for i in range(self.num_hidden_layers):
            window = self.layer_windows[i] if self.layer_windows else None
            mixer = MixerSpec.make(
                "attention",
                position=pos,
                n_heads=self.num_attention_heads,
                n_kv_heads=self.num_key_value_heads,
                head_dim=self.head_dim,
                bias=self.attention_bias,
                qk_norm=True,
                qk_norm_eps=self.rms_norm_eps,
                window=window,
                scale=None,
            )
            layers.append(
                LayerSpec(
                    prefix=f"model.layers.{i}",
                    mixer=mixer,
                    feed_forward=ff,
                    mixer_norm=norm,
                    ff_norm=norm,
                    arrangement="pre_norm",
                )
            )
        return ModelSpec(
            architecture=ARCHITECTURE,
            hidden=self.hidden_size,
            vocab=self.vocab_size,
            max_position=self.max_position_embeddings,
            layers=tuple(layers),
            schedule=tuple(ScheduleEntry(i) for i in range(self.num_hidden_layers)),
            final_norm=norm,
            tie_embeddings=self.tie_word_embeddings,
            stop_tokens=self.eos_token_ids,
        )

    def flat(self) -> dict:
        return asdict(self)
