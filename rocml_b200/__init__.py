"""rocml_b200: a small, whole model library for one GPU.

From a model folder (config.json + model.safetensors) to generated tokens: typed
configuration and registry, weights by tensor name, layers put together from parts, a paged
cache with a slot per sequence, one step function, a generation loop, sampling, and
hand-written CUDA kernels for sm_100a underneath.  One architecture is registered, the dense
Qwen3 decoder; another is added by registering its configuration (and any new parts).
"""
from . import config  # registers the built-in architecture
from . import parts   # registers the built-in parts
from .errors import (
    CacheError, CacheFull, ConfigError, ContextOverflow, ExtensionMissing, KernelError,
    MemoryBudget, ModelFileMissing, RocmlError, SafetensorsError, UnknownModel, UnsupportedArchitecture, WeightsError,
)
from .engine import Engine, Model, StepEntry
from .engine.generate import Completion, GenerateStats, Request, generate
from .sampling import SamplingParams

__version__ = "0.1.0"

__all__ = [
    "config", "parts", "Engine", "Model", "StepEntry", "Completion", "GenerateStats", "Request",
    "generate", "SamplingParams", "CacheError", "CacheFull", "ConfigError",
    "ContextOverflow", "ExtensionMissing", "KernelError", "MemoryBudget", "ModelFileMissing", "RocmlError",
    "SafetensorsError", "UnknownModel", "UnsupportedArchitecture", "WeightsError",
]
