"""Random weights: a model folder written from a configuration and a seed.

The reference has no such mode (it always opens a checkpoint); benchmarks and
tests here need one because no checkpoint can be fetched.  Distributions: linear
weights and embeddings N(0, 0.02); norm scales 1 + N(0, 0.1); biases N(0, 0.02).
Each tensor's values depend only on (seed, tensor name), never on the order in
which tensors are produced, and are rounded to bfloat16 so that the 32-bit and
the bfloat16 paths see exactly the same numbers.
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Iterator, Sequence, Tuple

import torch

from .decl import TensorDecl
from .safetensors_io import write_safetensors


def _seed_for(seed: int, name: str) -> int:
    h = hashlib.blake2b(f"{seed}:{name}".encode("utf-8"), digest_size=8).digest()
    return int.from_bytes(h, "little") & ((1 << 62) - 1)


def random_tensor(decl: TensorDecl, seed: int, device="cpu", dtype=torch.bfloat16) -> torch.Tensor:
    g = torch.Generator(device=device)
    g.manual_seed(_seed_for(seed, decl.name))
    if decl.role == "int_table":
        return torch.randint(0, 1 << 15, decl.shape, generator=g, device=device, dtype=torch.int32)
    x = torch.randn(decl.shape, generator=g, device=device, dtype=torch.float32)
    if decl.role == "norm":
        x.mul_(0.1).add_(1.0)
    else:
        x.mul_(0.02)
    return x.to(dtype)


def random_tensors(decls: Sequence[TensorDecl], seed: int, device="cpu",
                   dtype=torch.bfloat16) -> Iterator[Tuple[str, torch.Tensor]]:
    for d in decls:
        yield d.name, random_tensor(d, seed, device, dtype)


def write_random_model(folder: str, config, seed: int, dtype=torch.bfloat16) -> str:
    """Write ``folder/config.json`` and ``folder/model.safetensors`` for ``config``
    (a typed configuration of a registered architecture).  Returns the folder."""
    from ..engine.model import declared_tensors  # late: avoids an import cycle

    os.makedirs(folder, exist_ok=True)
    spec = config.to_model_spec()
    decls = declared_tensors(spec)
    with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as f:
        json.dump(config.to_dict(), f, indent=1)
    layout = [(d.name, torch.int32 if d.role == "int_table" else dtype, d.shape) for d in decls]
    write_safetensors(
        os.path.join(folder, "model.safetensors"), layout, random_tensors(decls, seed, "cpu", dtype),
        metadata={"format": "pt", "seed": str(seed)},
    )
    return folder
