"""Weights from a model folder, by tensor name.

The model declares the tensors it needs (``TensorDecl``); the loader checks the
whole folder against the declaration first and raises ONE ``WeightsError`` that
lists every missing tensor, every unexpected tensor and every wrong shape.  A
folder whose only fault is tensors the model does not read (checkpoints often
carry a few: rotary tables, training leftovers) is loaded with one warning that
names them; ``strict=True`` makes that an error too.  Then the tensors move to
the device under the storage rule:

* ``bfloat16`` mode: floating tensors are kept in bfloat16 (float16 is converted);
  a tensor the file stores in 32-bit stays 32-bit; integer tables become int32.
* ``float32`` mode: every floating tensor is widened to float32 (exact for
  bfloat16 and float16 values).

The reference does the same job for GGUF: look each tensor up by name, check its
shape, convert, upload (rocml/src/weights/mod.rs:37-175, weights/layer.rs:34-64).
"""
from __future__ import annotations

import warnings
from typing import Callable, Dict, Iterable, Sequence

import torch

from ..errors import WeightsError
from .decl import TensorDecl
from .safetensors_io import ModelFiles

_FLOATS = (torch.float64, torch.float32, torch.float16, torch.bfloat16)
_INTS = (torch.int64, torch.int32, torch.int16, torch.int8, torch.uint8)


def storage_dtype(file_dtype: torch.dtype, mode: str, role: str) -> torch.dtype:
    if role == "int_table" or file_dtype in _INTS:
        return torch.int32
    if mode == "float32":
        return torch.float32
    if mode != "bfloat16":
        raise ValueError(f"dtype mode must be 'bfloat16' or 'float32', found {mode!r}")
    if file_dtype in (torch.float32, torch.float64):
        return torch.float32
    return torch.bfloat16


class UnexpectedTensors(UserWarning):
    """A model folder holds tensors that the model does not read."""


def check_against(decls: Sequence[TensorDecl], names: Iterable[str], shape_of: Callable[[str], tuple],
                  ignorable: Iterable[str] = (), strict: bool = False) -> None:
    """Raise one WeightsError listing everything that does not fit.  Unexpected tensors alone are a
    warning unless ``strict``."""
    have = set(names)
    want = {d.name: d for d in decls}
    ignorable = set(ignorable)
    missing = sorted(n for n in want if n not in have)
    unexpected = sorted(n for n in have if n not in want and n not in ignorable)
    wrong = []
    for n, d in want.items():
        if n in have and tuple(shape_of(n)) != tuple(d.shape):
            wrong.append((n, tuple(d.shape), tuple(shape_of(n))))
    if missing or wrong or (unexpected and strict):
        raise WeightsError(missing, unexpected, sorted(wrong))
    if unexpected:
        shown = ", ".join(unexpected[:8]) + (f", ... ({len(unexpected)} in all)" if len(unexpected) > 8 else "")
        warnings.warn(f"the folder holds tensors the model does not read: {shown}", UnexpectedTensors, stacklevel=3)


def load_tensors(folder: str, decls: Sequence[TensorDecl], mode: str, device,
                 ignorable: Iterable[str] = (), strict: bool = False) -> Dict[str, torch.Tensor]:
    """name -> device tensor for every declared tensor of the folder."""
    with ModelFiles(folder) as files:
        check_against(decls, files.names(), files.shape, ignorable, strict)
        bad_dtype = []
        for d in decls:
            ft = files.dtype(d.name)
            if d.role == "int_table":
                if ft not in _INTS:
                    bad_dtype.append(f"{d.name}: integer table stored as {ft}")
            elif ft not in _FLOATS:
                bad_dtype.append(f"{d.name}: stored as {ft}, expected a floating type")
        if bad_dtype:
            raise WeightsError(other=bad_dtype)
        out = {}
        on_gpu = torch.device(device).type == "cuda"
        for d in decls:
            ft = files.dtype(d.name)
            dt = storage_dtype(ft, mode, d.role)
            if on_gpu:
                # file -> pinned staging -> device by the library's own reader; a conversion, if the storage
                # rule asks for one, happens on the device
                with torch.cuda.device(device):
                    raw = torch.empty(files.shape(d.name), dtype=ft, device=device)
                    files.read_into(d.name, raw)
                    out[d.name] = raw if ft == dt else raw.to(dt)
            else:
                out[d.name] = files.tensor(d.name).to(device=device, dtype=dt, non_blocking=False).contiguous()
        return out
