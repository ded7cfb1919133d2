"""Typed configurations, the architecture registry and the catalog of short names."""
from .specs import (
    FeedForwardSpec, LayerSpec, MixerSpec, ModelSpec, NormSpec, PositionSpec, ScheduleEntry,
)
from .qwen3 import Qwen3Config, ARCHITECTURE as QWEN3_ARCHITECTURE
from .registry import (
    CATALOG, CatalogEntry, ResolvedModel, SamplingPreset, checkpoint_dir, config_from_dict,
    load_config, load_model_spec, register_architecture, registered_architectures, resolve,
)

register_architecture(QWEN3_ARCHITECTURE, Qwen3Config.from_dict)

__all__ = [
    "FeedForwardSpec", "LayerSpec", "MixerSpec", "ModelSpec", "NormSpec", "PositionSpec",
    "ScheduleEntry", "Qwen3Config", "QWEN3_ARCHITECTURE", "CATALOG", "CatalogEntry",
    "ResolvedModel", "SamplingPreset", "checkpoint_dir", "config_from_dict", "load_config",
    "load_model_spec", "register_architecture", "registered_architectures", "resolve",
]
