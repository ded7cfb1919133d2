"""RMSNorm, fused with the residual addition that precedes it."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import kernels
from ..config.specs import NormSpec
from ..weights.decl import TensorDecl
from .base import BuildEnv, DeferredNorm, Norm, register_norm


@register_norm("rmsnorm")
class RMSNorm(Norm):
    """x * rsqrt(mean(x^2) + eps) * w, statistics in 32-bit
    (rocml-kernels/kernels/rmsnorm.hip:18-41); the weight multiplies directly."""

    graph_safe = True

    def __init__(self, spec: NormSpec, size: int, env: BuildEnv):
        self.eps = float(spec.eps)
        self.size = size
        self.env = env
        self.weight: Optional[torch.Tensor] = None

    def declare(self, prefix: str) -> List[TensorDecl]:
        return [TensorDecl(f"{prefix}.weight", (self.size,), "norm")]

    def load(self, tensors: Dict[str, torch.Tensor], prefix: str) -> None:
        self.weight = tensors[f"{prefix}.weight"]

    def weight_bytes(self) -> int:
        if self.weight is None:
            return self.size * (4 if self.env.mode == "float32" else 2)
        return self.weight.numel() * self.weight.element_size()

    def workspace_bytes(self, n_tokens: int) -> int:
        return n_tokens * self.size * (4 if self.env.mode == "float32" else 2)

    deferrable = True     # a product's epilogue can prepare this norm's input (see parts.base.DeferredNorm)

    def forward(self, resid, delta, n_rows: Optional[int] = None, rows=None, write_back=True):
        if isinstance(delta, DeferredNorm):
            # the part before has added its result into the residual already
            if delta.norm is self and rows is None:
                return delta            # and prepared this norm's rows: nothing to launch
            delta = None
        n = (rows.numel() if rows is not None else resid.shape[0]) if n_rows is None else n_rows
        out = torch.empty((n, self.size), dtype=self.env.act_dtype, device=resid.device)
        if delta is None:
            write_back = False          # nothing is added: the residual stays as it is
        kernels.add_rmsnorm(resid, delta, self.weight, self.eps, out, rows=rows, n_rows=n, write_back=write_back)
        return out
