"""Sampling parameters and the host-side random stream."""
from __future__ import annotations

from dataclasses import dataclass, replace
from typing import Optional

_MASK = (1 << 64) - 1


@dataclass(frozen=True)
class SamplingParams:
    """The reference's fields and defaults (rocml/src/sample.rs:16-41): temperature <= 0 is greedy
    and ignores the rest; top_k None keeps every token; top_p None disables the nucleus;
    repeat_penalty None disables the penalty, which otherwise looks at the last
    ``repeat_penalty_window`` ids of prompt + generated tokens."""

    temperature: float = 0.0
    top_k: Optional[int] = None
    top_p: Optional[float] = None
    seed: int = 0
    repeat_penalty: Optional[float] = None
    repeat_penalty_window: int = 64

    @property
    def is_greedy(self) -> bool:
        return self.temperature <= 0.0

    def merged(self, temperature=None, top_k=None, top_p=None, seed=None) -> "SamplingParams":
        """Explicit values win over this preset (rocml-cli/src/common.rs:167-176)."""
        return replace(
            self,
            temperature=self.temperature if temperature is None else temperature,
            top_k=self.top_k if top_k is None else top_k,
            top_p=self.top_p if top_p is None else top_p,
            seed=self.seed if seed is None else seed,
        )


class XorShift64Star:
    """The reference's generator (rocml/src/sample.rs:56-83): xorshift64*, seed 0 remapped to
    0x9E3779B97F4A7C15, uniform float = top 24 bits / 2^24."""

    def __init__(self, seed: int):
        seed &= _MASK
        self.state = 0x9E3779B97F4A7C15 if seed == 0 else seed

    def next_u64(self) -> int:
        x = self.state
        x ^= x >> 12
        x ^= (x << 25) & _MASK
        x ^= x >> 27
        self.state = x
        return (x * 0x2545F4914F6CDD1D) & _MASK

    def next_f32(self) -> float:
        return (self.next_u64() >> 40) / float(1 << 24)
