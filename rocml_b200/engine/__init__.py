"""Model assembly, the step function, generation and trace replay."""
from .batch import BatchBuffers, HostBatch, StepBatch, pack_entries
from .model import Model, declared_tensors
from .engine import Engine, StepEntry

__all__ = ["BatchBuffers", "HostBatch", "StepBatch", "pack_entries", "Model", "declared_tensors",
           "Engine", "StepEntry"]
