"""Gated feed-forward: down(act(gate(x)) * up(x)) (rocml/src/forward/ffn.rs:57-107)."""
from __future__ import annotations

from typing import Dict, List

import torch

from .. import kernels
from ..config.specs import FeedForwardSpec, tensor_names
from ..errors import ConfigError
from ..weights.decl import TensorDecl
from .base import BuildEnv, DeferredNorm, FeedForward, register_feed_forward
from .linear import GATED_PAIR_MAX_ROWS, Linear


# Tensor-name stems by role, unless the spec's ``names`` says otherwise (rocml/src/weights/layer.rs:59-62).
TENSOR_NAMES = {"gate": "gate_proj", "up": "up_proj", "down": "down_proj"}


@register_feed_forward("gated_mlp")
class GatedMLP(FeedForward):
    """gate and up are one stacked product [T, 2I]; SiLU(gate) * up -> [T, I]; down -> [T, H].
    The activation is a parameter; 'silu' (g / (1 + exp(-g)), rocml-kernels/kernels/
    silu_mul.hip:15-18) is the one built."""

    graph_safe = True

    def __init__(self, spec: FeedForwardSpec, hidden: int, env: BuildEnv):
        p = spec.params
        self.env = env
        self.hidden = hidden
        self.inter = int(p["intermediate"])
        act = p.get("activation", "silu")
        if act != "silu":
            raise ConfigError(f"activation {act!r} is not built (only 'silu')")
        bias = bool(p.get("bias", False))
        try:
            n = tensor_names(p, TENSOR_NAMES)
        except ValueError as e:
            raise ConfigError(f"gated_mlp: {e}") from None
        self.gate_up = Linear([n["gate"], n["up"]], [self.inter, self.inter], hidden, bias, env)
        self.down = Linear([n["down"]], [hidden], self.inter, bias, env)

    def declare(self, prefix: str) -> List[TensorDecl]:
        return self.gate_up.declare(prefix) + self.down.declare(prefix)

    def load(self, tensors: Dict[str, torch.Tensor], prefix: str) -> None:
        self.gate_up.load(tensors, prefix)
        self.down.load(tensors, prefix)
        if self.env.act_dtype == torch.bfloat16:
            self.gate_up.interleave_pairs()     # silu(gate) * up then happens inside the product

    def weight_bytes(self) -> int:
        return self.gate_up.weight_bytes() + self.down.weight_bytes()

    def workspace_bytes(self, n_tokens: int) -> int:
        """gate | up, their gated product and the delta (as partial sums: up to 8 of each for few tokens)."""
        esz = 4 if self.env.mode == "float32" else 2
        parts = 8 if n_tokens <= 128 else 1
        return n_tokens * (2 * self.inter * (4 * parts if parts > 1 else esz) + self.inter * esz + self.hidden * 4 * parts)

    def cost(self, q_lens, kv_lens):
        T = sum(q_lens)
        a, b = self.gate_up.cost(T), self.down.cost(T)
        return a[0] + b[0], a[1] + b[1]

    can_sink = True        # forward() accepts sink=ResidualSink (see parts.base)

    def takes_deferred(self, batch) -> bool:
        """Whether forward() can be handed a DeferredNorm for this step: only the product of two blocks
        that applies the activation itself also applies the rows' 1/RMS."""
        T = batch.n_tokens
        return (self.gate_up.paired and T <= GATED_PAIR_MAX_ROWS and self.gate_up.weight.dtype == torch.bfloat16
                and self.gate_up._splits(T) == 2 and self.gate_up.k > 64)

    can_add_into = True    # forward() accepts add_into=residual (see parts.base)

    def forward(self, xn, batch, sink=None, add_into=None):
        T = batch.n_tokens
        dev, act = self.env.device, self.env.act_dtype
        h = None
        if isinstance(xn, DeferredNorm):
            h = self.gate_up.forward_gated_pair(xn.x, T, rowscale=xn.rowscale)
            if h is None:
                xn = xn.materialize()     # the kernel declined after all: the norm's own kernel, then as always
        if h is None and self.gate_up.paired and T > 128:
            # many tokens: the activation happens in the product's epilogue, hidden behind the next tile
            h = self.gate_up.forward_gated(xn, T)
        elif h is None and self.gate_up.paired:
            # few tokens, the sum over K in two halves: the activation happens where the halves meet
            h = self.gate_up.forward_gated_pair(xn, T)
        if h is None:
            # the product is split over K some other way, so the activation waits for the partial sums
            gu = self.gate_up.forward_auto(xn, T)      # [T, 2I] or [S, T, 2I] partial sums
            h = torch.empty((T, self.inter), dtype=act, device=dev)
            kernels.silu_mul(gu, h, paired=self.gate_up.paired)
        if sink is not None:
            deferred = self.down.forward_residual(h, T, sink)
            if deferred is not None:
                return deferred
        if add_into is not None and self.down.forward_add(h, T, add_into):
            return None
        return self.down.forward_delta(h, T)
