"""What a model says about the tensors it needs."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Tuple


@dataclass(frozen=True)
class TensorDecl:
    """One tensor of the weight files.

    role: "matrix" (a linear weight or an embedding table, [out, in]),
    "norm" (a norm's scale vector), "bias", "int_table" (integer table), or
    "state" (anything else a part defines; initialised like a matrix).
    """

    name: str
    shape: Tuple[int, ...]
    role: str = "matrix"
