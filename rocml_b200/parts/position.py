"""Position encodings.  A mixer's fused kernel rotates queries and keys by the angles
pos * inv_freq[i]; the encoding owns that table, so another encoding (a partial rotation,
another base, scaled frequencies) is another table, not another kernel."""
from __future__ import annotations

import torch

from ..config.specs import PositionSpec
from ..errors import ConfigError
from .base import BuildEnv, PositionEncoding, register_position


@register_position("none")
class NoPosition(PositionEncoding):
    graph_safe = True

    def __init__(self, spec: PositionSpec, head_dim: int, env: BuildEnv):
        self.inv_freq = None
        self.rot_dim = 0

    def cos_sin(self, batch):
        return None


@register_position("rope_neox")
class RotaryNeox(PositionEncoding):
    """Rotate-half rotary embedding: inv_freq[i] = theta^(-2i / rot_dim) for i < rot_dim / 2,
    pairs (i, i + rot_dim / 2) (rocml-kernels/kernels/rope.hip:18-33).  The exponent and the
    power are evaluated in double precision and rounded once to float32; the angle
    pos * inv_freq and its sine and cosine are 32-bit, in the kernel."""

    graph_safe = True

    def __init__(self, spec: PositionSpec, head_dim: int, env: BuildEnv):
        rot = head_dim if spec.rot_dim is None else int(spec.rot_dim)
        if rot <= 0 or rot % 2 or rot > head_dim:
            raise ConfigError(f"rotary dimension {rot} must be even and at most the head size {head_dim}")
        if not spec.theta > 0:
            raise ConfigError(f"rotary base must be positive, found {spec.theta}")
        self.rot_dim = rot
        self.theta = float(spec.theta)
        i = torch.arange(rot // 2, dtype=torch.float64)
        inv = torch.pow(torch.tensor(float(spec.theta), dtype=torch.float64), -2.0 * i / rot)
        self.inv_freq = inv.to(torch.float32).to(env.device)

    def cos_sin(self, batch):
        """(cos, sin) of every token's angles for this step, computed once and shared by all the
        layers that use this encoding with the same table."""
        from .. import kernels
        key = ("rope_neox", self.rot_dim, self.theta)      # layers with the same encoding share the table
        if key not in batch.scratch:
            batch.scratch[key] = kernels.rope_table(batch.positions, self.inv_freq, batch.n_tokens)
        return batch.scratch[key]
