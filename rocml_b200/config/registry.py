"""One registry from an architecture's name to its configuration class, and the
catalog of short model names.

``resolve`` follows the reference's rule (rocml/src/registry/mod.rs:42-84,
123-127): something that looks like a path bypasses the catalog and brings no
defaults; a short name is looked up, an unknown one fails with the list of known
names, and a known one whose folder is absent fails naming the path and the
remedies.  Nothing is downloaded.  The catalog (names, sizes, default context,
default sampling: rocml/src/registry/catalog.rs:44-51,216-258) is data in
``catalog.json``.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Callable, Dict, Optional

from ..errors import ConfigError, ModelFileMissing, UnknownModel, UnsupportedArchitecture
from .specs import ModelSpec

# architecture name -> callable(dict) -> typed config with .to_model_spec() and .to_dict()
_ARCHITECTURES: Dict[str, Callable] = {}


def register_architecture(name: str, config_from_dict: Callable) -> None:
    """Make ``name`` (the string in config.json's ``architectures``) loadable.

    ``config_from_dict(d)`` returns the typed configuration; it must offer
    ``to_model_spec() -> ModelSpec`` and ``to_dict() -> dict``.
    """
    _ARCHITECTURES[name] = config_from_dict


def registered_architectures():
    return tuple(sorted(_ARCHITECTURES))


def config_from_dict(d: dict):
    archs = d.get("architectures") or []
    if not archs:
        raise ConfigError("config.json lacks 'architectures'")
    name = archs[0]
    if name not in _ARCHITECTURES:
        raise UnsupportedArchitecture(name, registered_architectures())
    return _ARCHITECTURES[name](d)


def load_config(folder: str):
    """Typed configuration of the model folder, chosen by config.json's architecture."""
    path = os.path.join(folder, "config.json") if os.path.isdir(folder) else folder
    if not os.path.isfile(path):
        raise ModelFileMissing(f"no config.json at {path}")
    try:
        with open(path, "r", encoding="utf-8") as f:
            d = json.load(f)
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path} is not valid JSON: {e}") from e
    if not isinstance(d, dict):
        raise ConfigError(f"{path} does not hold a JSON object")
    cfg = config_from_dict(d)
    gen = os.path.join(os.path.dirname(path), "generation_config.json")
    extra_stop = ()
    if os.path.isfile(gen):
        try:
            with open(gen, "r", encoding="utf-8") as f:
                g = json.load(f)
            e = g.get("eos_token_id")
            extra_stop = tuple(e) if isinstance(e, list) else ((e,) if isinstance(e, int) else ())
        except (json.JSONDecodeError, OSError):
            extra_stop = ()
    return cfg, extra_stop


def load_model_spec(folder: str) -> ModelSpec:
    cfg, extra_stop = load_config(folder)
    spec = cfg.to_model_spec()
    if extra_stop:
        stops = tuple(dict.fromkeys(spec.stop_tokens + extra_stop))
        spec = ModelSpec(**{**spec.__dict__, "stop_tokens": stops})
    return spec


# ---- catalog of short names ---------------------------------------------------

@dataclass(frozen=True)
class SamplingPreset:
    temperature: float = 0.0
    top_k: Optional[int] = None
    top_p: Optional[float] = None
    seed: int = 0


@dataclass(frozen=True)
class CatalogEntry:
    name: str
    folder: str
    default_ctx: int
    sampling: SamplingPreset
    config: dict

    @property
    def architecture(self) -> str:
        return self.config["architectures"][0]


@dataclass(frozen=True)
class ResolvedModel:
    path: str
    entry: Optional[CatalogEntry]  # None for a path: no defaults


def _read_catalog() -> Dict[str, CatalogEntry]:
    with open(os.path.join(os.path.dirname(__file__), "catalog.json"), "r", encoding="utf-8") as f:
        raw = json.load(f)
    presets = {k: SamplingPreset(**v) for k, v in raw["sampling_presets"].items()}
    out = {}
    for name, e in raw["models"].items():
        out[name] = CatalogEntry(name, e["folder"], int(e["default_ctx"]), presets[e["sampling"]], e["config"])
    return out


CATALOG: Dict[str, CatalogEntry] = _read_catalog()


def checkpoint_dir() -> str:
    """Where named models are looked for: $ROCML_CHECKPOINT_DIR, else ~/checkpoints
    (rocml/src/registry/mod.rs:158-167)."""
    env = os.environ.get("ROCML_CHECKPOINT_DIR")
    if env:
        return env
    return os.path.join(os.path.expanduser("~"), "checkpoints")


def is_path_like(name_or_path: str) -> bool:
    return os.sep in name_or_path or name_or_path.startswith(".") or os.path.isdir(name_or_path)


def resolve(name_or_path: str, must_exist: bool = True) -> ResolvedModel:
    if is_path_like(name_or_path):
        return ResolvedModel(name_or_path, None)
    entry = CATALOG.get(name_or_path)
    if entry is None:
        raise UnknownModel(name_or_path, sorted(CATALOG))
    path = os.path.join(checkpoint_dir(), entry.folder)
    if must_exist and not os.path.isfile(os.path.join(path, "config.json")):
        raise ModelFileMissing(
            f"model {entry.name!r} is not present: expected a folder with config.json and "
            f"model.safetensors at {path}. Put the checkpoint there (set ROCML_CHECKPOINT_DIR to "
            f"move the search root), or generate random weights of this size with "
            f"`python -m rocml_b200 generate --model {entry.name} --random`."
        )
    return ResolvedModel(path, entry)
