"""Reading and writing safetensors files, without any dependency.

Format: an 8-byte little-endian header length, a JSON header mapping each tensor
name to ``{"dtype", "shape", "data_offsets": [begin, end]}`` (offsets relative to
the end of the header), then the raw little-endian data.  The reader maps the
file into memory and hands out zero-copy CPU tensors; the writer streams tensors
one at a time, so a model larger than host memory's spare room can be written.

This takes the place of the reference's GGUF reader
(rocml-core/src/gguf/mod.rs:47-236): open, look a tensor up by name, know its
shape and type, and fail with a typed error on a truncated or malformed file.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, Iterator, List, Tuple

import torch

from ..errors import ModelFileMissing, SafetensorsError

_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8,
    "U8": torch.uint8, "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}
_MAX_HEADER = 100 * 1024 * 1024


def _numel(shape) -> int:
    n = 1
    for s in shape:
        n *= int(s)
    return n


class SafetensorsFile:
    """One open safetensors file."""

    def __init__(self, path: str):
        if not os.path.isfile(path):
            raise ModelFileMissing(f"no safetensors file at {path}")
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsError(f"{path}: file of {size} bytes is too short for a header")
        self._f = open(path, "rb")
        (hlen,) = struct.unpack("<Q", self._f.read(8))
        if hlen > _MAX_HEADER or 8 + hlen > size:
            raise SafetensorsError(
                f"{path}: header length {hlen} does not fit the file of {size} bytes (truncated?)"
            )
        try:
            header = json.loads(self._f.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON: {e}") from e
        if not isinstance(header, dict):
            raise SafetensorsError(f"{path}: header is not a JSON object")
        self.metadata = header.pop("__metadata__", {}) or {}
        self._base = 8 + hlen
        self._entries: Dict[str, Tuple[torch.dtype, Tuple[int, ...], int, int]] = {}
        data_size = size - self._base
        for name, e in header.items():
            try:
                dtype = _DTYPES[e["dtype"]]
                shape = tuple(int(s) for s in e["shape"])
                b, en = (int(x) for x in e["data_offsets"])
            except (KeyError, TypeError, ValueError) as err:
                raise SafetensorsError(f"{path}: bad entry for tensor {name!r}: {err!r}") from err
            want = _numel(shape) * torch.empty((), dtype=dtype).element_size()
            if en - b != want or b < 0 or en > data_size:
                raise SafetensorsError(
                    f"{path}: tensor {name!r} spans bytes [{b}, {en}) but shape {list(shape)} "
                    f"needs {want} and the data section holds {data_size} (truncated?)"
                )
            self._entries[name] = (dtype, shape, b, en)
        self._mm = None
        self._native = None

    def names(self) -> List[str]:
        return list(self._entries)

    def __contains__(self, name: str) -> bool:
        return name in self._entries

    def shape(self, name: str) -> Tuple[int, ...]:
        return self._entries[name][1]

    def dtype(self, name: str) -> torch.dtype:
        return self._entries[name][0]

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor viewing the mapped file (copy-on-write; do not keep it after close)."""
        dtype, shape, b, en = self._entries[name]
        if self._mm is None:
            self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_COPY)
        n = _numel(shape)
        if n == 0:
            return torch.empty(shape, dtype=dtype)
        t = torch.frombuffer(self._mm, dtype=dtype, count=n, offset=self._base + b)
        return t.view(shape)

    def read_into(self, name: str, dst: torch.Tensor) -> None:
        """Fill ``dst`` (a contiguous tensor of the tensor's shape and stored type, on a CUDA device) with the
        tensor's bytes, through the library's own reader: file -> pinned staging -> device on the current
        stream, without a Python object in between (``csrc/safetensors_reader.cu``)."""
        dtype, shape, b, en = self._entries[name]
        if dst.dtype != dtype or tuple(dst.shape) != shape or not dst.is_contiguous() or not dst.is_cuda:
            raise SafetensorsError(f"{self.path}: destination for {name!r} must be a contiguous CUDA tensor {dtype} {list(shape)}")
        if self._native is None:
            self._native = NativeReader(self.path)
        self._native.read(name, dst, en - b)

    def close(self) -> None:
        # Tensors handed out keep the mapping alive through the buffer protocol.
        self._mm = None
        self._f.close()
        if self._native is not None:
            self._native.close()
            self._native = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


class NativeReader:
    """The library's reader of one safetensors file (``csrc/safetensors_reader.cu``): it parses and checks the
    header itself, and copies a tensor's bytes to host or device memory."""

    def __init__(self, path: str):
        import ctypes
        from ..csrc.build import library
        self._c = ctypes
        lib = self._lib = library()
        if not getattr(lib, "_st_sigs", False):
            vp, i, ll = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
            lib.rb_st_open.argtypes = [ctypes.c_char_p, ctypes.c_char_p, i]
            lib.rb_st_open.restype = vp
            lib.rb_st_count.argtypes = [vp]
            lib.rb_st_entry.argtypes = [vp, i, ctypes.POINTER(ctypes.c_char_p), ctypes.POINTER(ctypes.c_char_p),
                                        ctypes.POINTER(i), ctypes.POINTER(ll), ctypes.POINTER(ll)]
            lib.rb_st_metadata_count.argtypes = [vp]
            lib.rb_st_metadata.argtypes = [vp, i, ctypes.POINTER(ctypes.c_char_p), ctypes.POINTER(ctypes.c_char_p)]
            lib.rb_st_read.argtypes = [vp, i, vp, ll, i, vp]
            lib.rb_st_close.argtypes = [vp]
            lib.rb_st_close.restype = None
            lib._st_sigs = True
        err = ctypes.create_string_buffer(1024)
        self._h = lib.rb_st_open(os.fsencode(path), err, len(err))
        if not self._h:
            raise SafetensorsError(err.value.decode("utf-8", "replace"))
        self.path = path
        self.entries: Dict[str, Tuple[int, str, Tuple[int, ...], int]] = {}     # name -> (index, dtype, shape, bytes)
        name, dtype = ctypes.c_char_p(), ctypes.c_char_p()
        rank, nbytes, shape = ctypes.c_int(), ctypes.c_longlong(), (ctypes.c_longlong * 8)()
        for k in range(lib.rb_st_count(self._h)):
            if lib.rb_st_entry(self._h, k, ctypes.byref(name), ctypes.byref(dtype), ctypes.byref(rank), shape,
                               ctypes.byref(nbytes)) != 0:
                self.close()
                raise SafetensorsError(f"{path}: a tensor of more than 8 dimensions")
            self.entries[name.value.decode("utf-8")] = (k, dtype.value.decode("ascii"), tuple(shape[:rank.value]), nbytes.value)
        self.metadata = {}
        key, value = ctypes.c_char_p(), ctypes.c_char_p()
        for k in range(lib.rb_st_metadata_count(self._h)):
            lib.rb_st_metadata(self._h, k, ctypes.byref(key), ctypes.byref(value))
            self.metadata[key.value.decode("utf-8")] = value.value.decode("utf-8")

    def read(self, name: str, dst: torch.Tensor, nbytes: int) -> None:
        index, _, _, have = self.entries[name]
        if have != nbytes or dst.numel() * dst.element_size() != nbytes:
            raise SafetensorsError(f"{self.path}: tensor {name!r} holds {have} bytes, asked for {nbytes}")
        if dst.is_cuda:
            stream = self._c.c_void_p(torch._C._cuda_getCurrentRawStream(dst.device.index or 0))
            rc = self._lib.rb_st_read(self._h, index, self._c.c_void_p(dst.data_ptr()), nbytes, 1, stream)
        else:
            rc = self._lib.rb_st_read(self._h, index, self._c.c_void_p(dst.data_ptr()), nbytes, 0, None)
        if rc != 0:
            raise SafetensorsError(f"{self.path}: reading tensor {name!r} failed (code {rc})")

    def close(self) -> None:
        if self._h:
            self._lib.rb_st_close(self._h)
            self._h = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


def write_safetensors(path: str, layout: Iterable[Tuple[str, torch.dtype, Tuple[int, ...]]],
                      tensors: Iterator[Tuple[str, torch.Tensor]], metadata: Dict[str, str] = None) -> None:
    """Write ``path``.  ``layout`` lists (name, dtype, shape) in file order; ``tensors``
    yields (name, tensor) in the same order, one at a time."""
    header = {}
    off = 0
    order = []
    for name, dtype, shape in layout:
        nbytes = _numel(shape) * torch.empty((), dtype=dtype).element_size()
        header[name] = {"dtype": _NAMES[dtype], "shape": list(shape), "data_offsets": [off, off + nbytes]}
        off += nbytes
        order.append((name, dtype, tuple(shape)))
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * (-len(blob) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        it = iter(tensors)
        for name, dtype, shape in order:
            got_name, t = next(it)
            if got_name != name or t.dtype != dtype or tuple(t.shape) != shape:
                raise SafetensorsError(
                    f"writer: expected {name} {dtype} {list(shape)}, got {got_name} {t.dtype} {list(t.shape)}"
                )
            t = t.detach().cpu().contiguous()
            f.write(t.view(torch.uint8).numpy().tobytes() if t.numel() else b"")
    os.replace(tmp, path)


def save_state_dict(path: str, state: Dict[str, torch.Tensor], metadata: Dict[str, str] = None) -> None:
    layout = [(k, v.dtype, tuple(v.shape)) for k, v in state.items()]
    write_safetensors(path, layout, iter(state.items()), metadata)


class ModelFiles:
    """All tensors of a model folder: ``model.safetensors``, or the shards that
    ``model.safetensors.index.json`` lists."""

    def __init__(self, folder: str):
        self.folder = folder
        single = os.path.join(folder, "model.safetensors")
        index = os.path.join(folder, "model.safetensors.index.json")
        self._files: List[SafetensorsFile] = []
        self._where: Dict[str, SafetensorsFile] = {}
        duplicates = []
        if os.path.isfile(single):
            paths = [single]
        elif os.path.isfile(index):
            try:
                with open(index, "r", encoding="utf-8") as f:
                    weight_map = json.load(f)["weight_map"]
            except (json.JSONDecodeError, KeyError, TypeError) as e:
                raise SafetensorsError(f"{index}: malformed shard index: {e!r}") from e
            paths = [os.path.join(folder, p) for p in sorted(set(weight_map.values()))]
        else:
            raise ModelFileMissing(f"no model.safetensors (or shard index) in {folder}")
        for p in paths:
            sf = SafetensorsFile(p)
            self._files.append(sf)
            for name in sf.names():
                if name in self._where:
                    duplicates.append(name)
                self._where[name] = sf
        if duplicates:
            raise SafetensorsError(f"{folder}: tensors stored in more than one shard: {sorted(duplicates)}")

    def names(self) -> List[str]:
        return list(self._where)

    def __contains__(self, name: str) -> bool:
        return name in self._where

    def shape(self, name: str):
        return self._where[name].shape(name)

    def dtype(self, name: str):
        return self._where[name].dtype(name)

    def tensor(self, name: str) -> torch.Tensor:
        return self._where[name].tensor(name)

    def read_into(self, name: str, dst: torch.Tensor) -> None:
        self._where[name].read_into(name, dst)

    def close(self):
        for f in self._files:
            f.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
