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

import functools
from typing import Dict, List, Optional, Sequence

import torch

from .. import kernels
from ..profile import profiler as _profiler
from ..errors import KernelError
from ..weights.decl import TensorDecl
from .base import BuildEnv, DeferredNorm


_SM_COUNT = {}

# The gated pair product (two K halves as a cluster, SiLU where they meet) beats the plain product
# followed by the activation kernel up to this many rows; its 32-row tiles are slower than the two
# kernels (51-57 us against 38-40 for a 24,576 x 4,096 weight).
GATED_PAIR_MAX_ROWS = 16


def _sm_count(device) -> int:
    key = torch.device(device).index or 0
    if key not in _SM_COUNT:
        _SM_COUNT[key] = torch.cuda.get_device_properties(device).multi_processor_count
    return _SM_COUNT[key]


def _labelled(fn):
    """While a profiler is active the kernels a product launches carry the weight's name as their label."""
    @functools.wraps(fn)
    def inner(self, *args, **kwargs):
        prof = _profiler.ACTIVE
        if prof is None:
            return fn(self, *args, **kwargs)
        with prof.scope(op=self.label):
            return fn(self, *args, **kwargs)
    return inner


class Linear:
    def __init__(self, names: Sequence[str], out_features: Sequence[int], in_features: int, bias: bool,
                 env: BuildEnv):
        """``names`` are the tensor-name stems stacked along out (e.g. q_proj, k_proj, v_proj)."""
        self.names = list(names)
        self.label = "+".join(n.rsplit(".", 1)[-1] for n in self.names)
        self.outs = list(out_features)
        self.n = sum(self.outs)
        self.k = in_features
        self.has_bias = bias
        self.env = env
        self.weight: Optional[torch.Tensor] = None
        self.bias: Optional[torch.Tensor] = None  # float32: widening is exact, the vector is tiny
        self.paired = False

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

    def interleave_pairs(self) -> bool:
        """For a stack of two equally wide projections (gate, up): reorder the rows so that blocks
        of 16 gate rows alternate with the 16 up rows of the same outputs.  The tensor-core
        product can then apply silu(gate) * up in its epilogue (``forward_gated``).  Returns False,
        and changes nothing, when the sizes or types do not allow it."""
        if len(self.outs) != 2 or self.outs[0] != self.outs[1] or self.outs[0] % 16 or self.k % 8 or \
                self.weight.dtype != torch.bfloat16 or not self.weight.is_cuda:
            return False
        half = self.outs[0]

        def mix(t):
            g, u = t[:half], t[half:]
            shape = (half // 16, 16) + tuple(t.shape[1:])
            return torch.stack([g.reshape(shape), u.reshape(shape)], dim=1).reshape(t.shape).contiguous()
        self.weight = mix(self.weight)
        if self.bias is not None:
            self.bias = mix(self.bias)
        self.paired = True
        return True

    @_labelled
    def forward_gated(self, x: torch.Tensor, m: int) -> torch.Tensor:
        """[M, N / 2] = silu(gate(x)) * up(x) in one kernel (needs ``interleave_pairs``)."""
        out = torch.empty((m, self.n // 2), dtype=torch.bfloat16, device=x.device)
        if not kernels.gemm_tcgen05(x, self.weight, out, self.bias, m, gated=True):
            raise KernelError("the gated matrix product refused a layout that interleave_pairs accepted")
        return out

    @_labelled
    def forward_gated_pair(self, x: torch.Tensor, m: int, rowscale=None) -> Optional[torch.Tensor]:
        """The same for few rows when the sum over K is split in two: the two halves' blocks form a
        cluster and the activation is applied where they meet, so no second kernel waits for partial
        sums.  None when this step's product is split otherwise or the kernel refuses."""
        if not (self.paired and self._tensor_core(x)) or self._splits(m) != 2 or m > GATED_PAIR_MAX_ROWS:
            return None
        out = torch.empty((m, self.n // 2), dtype=torch.bfloat16, device=x.device)
        return out if kernels.gemm_tcgen05_gated_pair(x, self.weight, out, self.bias, m, rowscale=rowscale) else None

    def residual_splits(self, m: int) -> int:
        """In how many parts ``forward_residual`` would split the sum over K for m rows (0: it would not
        take the step at all)."""
        if m > 64 or self.weight is None or self.weight.dtype != torch.bfloat16 or self.k % 8:
            return 0
        # clusters of 8: larger ones leave too few of them resident at once (a cluster needs all its
        # blocks on neighbouring multiprocessors)
        s = self._splits(m)
        s = 8 if s >= 8 else (4 if s >= 4 else 0)
        return s if s and self.k // 64 >= s else 0

    @_labelled
    def forward_residual(self, x: torch.Tensor, m: int, sink) -> Optional[DeferredNorm]:
        """sink.resid += x . W^T (+ bias) for a few rows, inside the product (the K splits exchange their
        parts through shared memory), together with what ``sink.norm`` needs: returns its deferred
        rows, or None when this step's product cannot be done that way (use ``forward_delta``)."""
        s = self.residual_splits(m)
        norm = sink.norm
        if not s or not self._tensor_core(x) or not getattr(norm, "deferrable", False) or norm.weight is None:
            return None
        xhat = torch.empty((m, self.n), dtype=torch.bfloat16, device=x.device)
        sumsq = torch.empty((((self.n + 127) // 128) * s, m), dtype=torch.float32, device=x.device)
        if not kernels.gemm_tcgen05_residual(x, self.weight, sink.resid, s, self.bias, norm.weight, xhat, sumsq, m):
            return None
        return DeferredNorm(xhat, sumsq, norm.eps, self.n, norm, sink.resid)

    @_labelled
    def forward_add(self, x: torch.Tensor, m: int, resid: torch.Tensor) -> bool:
        """resid += x . W^T (+ bias) for many rows, inside the product's epilogue.  False when this step's
        product cannot be done that way (use ``forward_delta``)."""
        if not self._tensor_core(x) or self._splits(m) != 1:
            return False
        return kernels.gemm_tcgen05_add(x, self.weight, resid, self.bias, m)

    def adopt(self, weight: torch.Tensor) -> None:
        """Use an existing tensor as the weight (a tied head reads the embedding table)."""
        if tuple(weight.shape) != (self.n, self.k):
            raise KernelError(f"tied weight has shape {tuple(weight.shape)}, expected {(self.n, self.k)}")
        self.weight = weight

    def weight_bytes(self) -> int:
        if self.weight is None:     # not loaded: the declared shape in the type the files would be kept in
            return self.n * self.k * (4 if self.env.mode == "float32" else 2)
        return self.weight.numel() * self.weight.element_size()

    def cost(self, m: int):
        """(bytes, operations) of the product with m rows: the weight once, 2 m n k."""
        return self.weight_bytes(), 2 * m * self.n * self.k

    def _tensor_core(self, x: torch.Tensor) -> bool:
        return x.dtype == torch.bfloat16 and self.weight.dtype == torch.bfloat16 and x.is_cuda

    @_labelled
    def forward(self, x: torch.Tensor, out: torch.Tensor, m: Optional[int] = None) -> torch.Tensor:
        """out[:M] = x[:M] . W^T (+ bias); ``out`` is [M, N] float32 or of x's type."""
        if self._tensor_core(x) and kernels.gemm_tcgen05(x, self.weight, out, self.bias, m):
            return out
        kernels.gemm_generic(x, self.weight, out, self.bias, m)
        return out

    def _splits(self, m: int) -> int:
        """How many ways the sum over K is split when few rows stream a large weight.  One
        thread block reads memory at a small fraction of the device's bandwidth, so the weight's
        row tiles (128 rows each) are multiplied by K splits until about two blocks per
        multiprocessor are in flight (more gains little and costs the consumer, which adds the
        partial sums); each split keeps at least five 64-wide K blocks, at most 8 splits, and the
        float32 partial results stay below a third of the weight's own bytes (they stay in the L2
        cache).  A product over a very deep K (24 or more K blocks left per split) is split twice
        as often, as long as all its blocks still fit on the device at once (four per
        multiprocessor) and the partial results stay below a sixth of the weight's bytes.  More
        than 128 rows: see below.  The count depends on the weight's shape, the step's row count
        and the device only."""
        if self.k % 8:
            return 1
        sms = _sm_count(self.env.device)
        if m > 128:
            # A few hundred rows: the output has fewer 128 x 256 tiles than the device has
            # multiprocessors, and each block would stream its share of the weight alone.  The sum over
            # K is split until the blocks fill one wave (measured at 160 to 1,024 rows: whenever tiles
            # times splits stays within the multiprocessors the split wins, up to 2.7 times; beyond, it
            # loses to the kernels for many rows).
            tiles = ((m + 127) // 128) * ((self.n + 255) // 256)
            s = min(sms // max(1, tiles), (self.k // 64) // 8, 8)
            return s if s >= 2 else 1
        tiles = (self.n + 127) // 128
        k_blocks = self.k // 64
        by_blocks = -(-2 * sms // tiles)
        by_depth = k_blocks // 5
        by_bytes = int(0.15 * self.k / max(m, 1))
        if m > 64 and tiles >= sms:
            return 1        # a block a multiprocessor already, and partial sums of many rows cost more than they gain (measured)
        s = max(1, min(by_blocks, by_depth, by_bytes, 8))
        if k_blocks // s >= 24 and 4 * s <= by_bytes and 2 * s * tiles <= 4 * sms:
            s *= 2
        return s

    def _splits_f32(self, x: torch.Tensor, m: int) -> int:
        """The same for the 32-bit product of at most 16 rows, in which a warp streams four weight rows: a
        narrow weight alone has too few rows to keep the memory busy, so the sum over K is cut until about 24
        warps a multiprocessor are at work (each part at least 1,024 values of k, at most 8 parts)."""
        if m > 16 or x.dtype != torch.float32 or self.weight is None or self.weight.dtype != torch.float32 \
                or self.k % 4 or not x.is_cuda:
            return 1
        warps = (self.n + 3) // 4
        return max(1, min(8, -(-24 * _sm_count(self.env.device) // warps), self.k // 1024))

    @_labelled
    def forward_delta(self, x: torch.Tensor, m: int) -> torch.Tensor:
        """The product as float32 [S, M, N]: S partial sums over K that the consumer adds in order
        (a delta for the residual stream, or the input of a kernel that takes partial sums)."""
        tc = self._tensor_core(x)
        S = self._splits(m) if tc else self._splits_f32(x, m)
        out = torch.empty((S, m, self.n), dtype=torch.float32, device=x.device)
        if tc and kernels.gemm_tcgen05(x, self.weight, out, self.bias, m):
            return out
        if not tc and S > 1:
            kernels.gemm_generic(x, self.weight, out, self.bias, m)
            return out
        if S > 1:
            out = out[:1]
        kernels.gemm_generic(x, self.weight, out[0], self.bias, m)
        return out

    def forward_auto(self, x: torch.Tensor, m: int) -> torch.Tensor:
        """The product in whichever form is cheapest for the step: [S, M, N] float32 partial sums
        when few rows stream the weight, else [M, N] in the activations' type."""
        if (self._tensor_core(x) and self._splits(m) > 1) or self._splits_f32(x, m) > 1:
            return self.forward_delta(x, m)
        out = torch.empty((m, self.n), dtype=x.dtype, device=x.device)
        return self.forward(x, out, m)
