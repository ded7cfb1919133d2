"""What a mixer asks of the cache."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch


@dataclass(frozen=True)
class KVRequirement:
    """Keys and values of every position (window None) or of the last ``window`` positions."""

    n_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class StateRequirement:
    """A tensor of fixed shape per sequence, zero when the sequence starts."""

    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32
