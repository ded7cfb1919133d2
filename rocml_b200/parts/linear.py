"""One linear weight and the matrix product with it.

y[M, N] = x[M, K] . W[N, K]^T (+ bias).  W is [out, in] row-major as the files store it
(rocml/src/weights/mod.rs:78-98); several projections that read the same input may be
stacked along ``out`` at load time (q|k|v, gate|up) so that one product serves them.
The product is chosen by the weight's own type: a 32-bit weight always goes through the
CUDA-core kernel with 32-bit FMA (never a tensor-core or reduced-precision mode); a
bfloat16 weight with bfloat16 activations goes to the tensor-core kernel when its sizes
allow and to the same CUDA-core kernel otherwise.  The reference makes the same split by
call shape: ``matvec`` for one token, ``matmul`` for many
(rocml/src/weights/linear.rs:142-156,172-207).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch

from .. import kernels
from ..errors import KernelError
from ..weights.decl import TensorDecl
from .base import BuildEnv


class Linear:
    def __init__(self, names: Sequence[str], out_features: Sequence[int], in_features: int, bias: bool,
                 env: BuildEnv):
        """``names`` are the tensor-name stems stacked along out (e.g. q_proj, k_proj, v_proj)."""
        self.names = list(names)
        self.outs = list(out_features)
        self.n = sum(self.outs)
        self.k = in_features
        self.has_bias = bias
        self.env = env
        self.weight: Optional[torch.Tensor] = None
        self.bias: Optional[torch.Tensor] = None  # float32: widening is exact, the vector is tiny

    def declare(self, prefix: str) -> List[TensorDecl]:
        out = []
        for name, n in zip(self.names, self.outs):
            out.append(TensorDecl(f"{prefix}{name}.weight", (n, self.k), "matrix"))
            if self.has_bias:
                out.append(TensorDecl(f"{prefix}{name}.bias", (n,), "bias"))
        return out

    def load(self, tensors: Dict[str, torch.Tensor], prefix: str) -> None:
        ws = [tensors[f"{prefix}{n}.weight"] for n in self.names]
        if len({w.dtype for w in ws}) != 1:
            ws = [w.float() for w in ws]  # stacked parts stored in different types: widen all
        self.weight = ws[0] if len(ws) == 1 else torch.cat(ws, dim=0).contiguous()
        if self.has_bias:
            self.bias = torch.cat([tensors[f"{prefix}{n}.bias"].float() for n in self.names]).contiguous()

    def adopt(self, weight: torch.Tensor) -> None:
        """Use an existing tensor as the weight (a tied head reads the embedding table)."""
        if tuple(weight.shape) != (self.n, self.k):
            raise KernelError(f"tied weight has shape {tuple(weight.shape)}, expected {(self.n, self.k)}")
        self.weight = weight

    def weight_bytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()

    def _tensor_core(self, x: torch.Tensor) -> bool:
        return x.dtype == torch.bfloat16 and self.weight.dtype == torch.bfloat16 and x.is_cuda

    def forward(self, x: torch.Tensor, out: torch.Tensor, m: Optional[int] = None) -> torch.Tensor:
        """out[:M] = x[:M] . W^T (+ bias); ``out`` is [M, N] float32 or of x's type."""
        if self._tensor_core(x) and kernels.gemm_tcgen05(x, self.weight, out, self.bias, m):
            return out
        kernels.gemm_generic(x, self.weight, out, self.bias, m)
        return out

    def forward_delta(self, x: torch.Tensor, m: int) -> torch.Tensor:
        """The product as a float32 delta [S, M, N] for the residual stream.  With few rows the
        sum over K is split S ways so that enough thread blocks stream the weight; the S partial
        results are added, in order, by the norm that consumes the delta.  S depends on the
        weight's shape and on whether the step is small, never on what else is in the batch."""
        S = 1
        if self._tensor_core(x) and m <= 128 and self.k % 8 == 0:
            tiles = (self.n + 127) // 128
            S = max(1, min(8, 148 // tiles, self.k // 512))
        delta = torch.empty((S, m, self.n), dtype=torch.float32, device=x.device)
        if self._tensor_core(x) and kernels.gemm_tcgen05(x, self.weight, delta, self.bias, m):
            return delta
        if S > 1:
            delta = delta[:1]
        kernels.gemm_generic(x, self.weight, delta[0], self.bias, m)
        return delta
