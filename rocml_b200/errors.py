"""Typed errors of the library.

Every failure a caller can provoke (a bad config.json, a model folder with the
wrong tensors, a cache that is full, a sequence past its context) is raised as
one of these, never as a bare assertion.  The classes mirror the reference's
error enum (rocml/src/error.rs:8-99): configuration, unsupported architecture,
unknown model, missing file, shape mismatch, context overflow, memory budget.
"""


class RocmlError(Exception):
    """Base class of every error this library raises on purpose."""


class ConfigError(RocmlError):
    """config.json is missing a key, or holds a value the architecture rejects."""


class UnsupportedArchitecture(RocmlError):
    """config.json names an architecture no model is registered for."""

    def __init__(self, found, known):
        self.found = found
        self.known = tuple(known)
        super().__init__(
            f"unsupported architecture {found!r}; registered: {', '.join(self.known) or '(none)'}"
        )


class UnknownModel(RocmlError):
    """A short model name that the catalog does not hold (rocml/src/registry/mod.rs:50-60)."""

    def __init__(self, name, known):
        self.name = name
        self.known = tuple(known)
        super().__init__(f"unknown model {name!r}; known names: {', '.join(self.known)}")


class ModelFileMissing(RocmlError):
    """A model folder lacks config.json or its safetensors file."""


class WeightsError(RocmlError):
    """The tensors of a model folder do not fit the model.

    One error lists everything that is wrong: tensors the model needs and the
    file lacks, tensors the file holds and the model does not know, and tensors
    whose shape differs.
    """

    def __init__(self, missing=(), unexpected=(), wrong_shape=(), other=()):
        self.missing = tuple(missing)
        self.unexpected = tuple(unexpected)
        self.wrong_shape = tuple(wrong_shape)  # (name, expected, found)
        self.other = tuple(other)
        lines = ["model weights do not match the model:"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        for name, want, got in self.wrong_shape:
            lines.append(f"  wrong shape: {name}: expected {list(want)}, found {list(got)}")
        for msg in self.other:
            lines.append(f"  {msg}")
        super().__init__("\n".join(lines))


class SafetensorsError(RocmlError):
    """A safetensors file is truncated or its header is malformed."""


class CacheError(RocmlError):
    """Misuse of the cache: a slot freed twice, an unknown slot, and the like."""


class CacheFull(CacheError):
    """No free slot or page is left for the request."""


class ContextOverflow(RocmlError):
    """A sequence would grow past the longest context the engine holds
    (rocml/src/error.rs:43, raised at rocml/src/forward/mod.rs:251-258)."""

    def __init__(self, requested, limit):
        self.requested = requested
        self.limit = limit
        super().__init__(f"context overflow: {requested} tokens requested, limit is {limit}")


class MemoryBudget(RocmlError):
    """The cache that was asked for does not fit the device memory that is left once the weights
    are resident (rocml/src/error.rs:46-54, checked at rocml/src/forward/mod.rs:145-161)."""

    def __init__(self, requested_tokens, suggested_tokens, breakdown):
        self.requested_tokens = requested_tokens
        self.suggested_tokens = suggested_tokens
        super().__init__(
            f"a cache of {requested_tokens} tokens does not fit the device: {breakdown}; "
            f"about {suggested_tokens} tokens would"
        )


class KernelError(RocmlError):
    """A CUDA kernel refused its sizes, or the CUDA runtime reported an error."""


class ExtensionMissing(RocmlError):
    """The compiled CUDA library is absent and cannot be built here."""
