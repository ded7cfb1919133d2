"""Grouped-query softmax attention over the paged cache.

Order, as in the reference (rocml/src/forward/attention.rs:56-244, attention_chunk.rs:
75-325): q, k, v projections (one stacked product) -> per-head RMSNorm of q and k, not v
-> position encoding of q and k -> k, v written to the cache -> attention of every query
over its sequence's keys at positions <= its own (and inside the window, if the layer has
one) -> output projection.  The result is returned as a delta for the residual stream.

Sizes and constants (heads, groups, head size, biases, q/k norm and its eps, window, scale)
are parameters; a layer that reads another layer's cache projects only q.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

from .. import kernels
from ..cache.requirements import KVRequirement
from ..config.specs import MixerSpec, tensor_names
from ..errors import ConfigError
from ..profile import scope
from ..weights.decl import TensorDecl
from .base import BuildEnv, DeferredNorm, Mixer, build_position, register_mixer
from .linear import Linear

# From this many tokens in a step the q | k | v projection normalises, rotates and caches in its own
# epilogue.  With fewer tokens a block has too few tiles to hide that epilogue behind the next tile's
# main loop, and the rotation kernel after a plain product is as fast or faster (measured at 1,024 and
# 2,048 tokens against 4,096).
PROMPT_FUSED_MIN_TOKENS = 4096

# Tensor-name stems by role, unless the spec's ``names`` says otherwise (the defaults are those of
# Hugging Face's Qwen3 checkpoints: rocml/src/weights/layer.rs:47-58 lists the same tensors under GGUF names).
TENSOR_NAMES = {"q": "q_proj", "k": "k_proj", "v": "v_proj", "o": "o_proj", "q_norm": "q_norm", "k_norm": "k_norm"}

DECODE_CHUNK = 64   # keys per split of decode attention (one page); fixed, so a row's sums never depend on the batch


@register_mixer("attention")
class Attention(Mixer):
    graph_safe = True

    def __init__(self, spec: MixerSpec, hidden: int, env: BuildEnv):
        p = spec.params
        self.env = env
        self.hidden = hidden
        self.nq = int(p["n_heads"])
        self.nkv = int(p["n_kv_heads"])
        self.hd = int(p["head_dim"])
        if self.nq <= 0 or self.nkv <= 0 or self.nq % self.nkv:
            raise ConfigError(f"{self.nq} query heads cannot be grouped over {self.nkv} key/value heads")
        if self.hd % 16 or self.hd > 256:
            raise ConfigError(f"head size {self.hd} is not supported: multiples of 16 up to 256")
        self.bias = bool(p.get("bias", False))
        self.qk_norm = bool(p.get("qk_norm", False))
        self.qk_norm_eps = float(p.get("qk_norm_eps", 1e-6))
        self.window = p.get("window")
        self.scale = float(p["scale"]) if p.get("scale") is not None else 1.0 / math.sqrt(self.hd)
        self.shares_cache = bool(p.get("shares_cache", False))  # set by the model for a reading layer
        self.position = build_position(spec.position, self.hd, env)
        qd, kvd = self.nq * self.hd, self.nkv * self.hd
        try:
            self.names = n = tensor_names(p, TENSOR_NAMES)
        except ValueError as e:
            raise ConfigError(f"attention: {e}") from None
        if self.shares_cache:
            self.qkv = Linear([n["q"]], [qd], hidden, self.bias, env)
        else:
            self.qkv = Linear([n["q"], n["k"], n["v"]], [qd, kvd, kvd], hidden, self.bias, env)
        self.o = Linear([n["o"]], [hidden], qd, self.bias, env)
        self.q_norm_w: Optional[torch.Tensor] = None
        self.k_norm_w: Optional[torch.Tensor] = None

    def cache_requirement(self):
        return KVRequirement(self.nkv, self.hd, self.window)

    def declare(self, prefix: str) -> List[TensorDecl]:
        out = self.qkv.declare(prefix) + self.o.declare(prefix)
        if self.qk_norm:
            out.append(TensorDecl(f"{prefix}{self.names['q_norm']}.weight", (self.hd,), "norm"))
            if not self.shares_cache:
                out.append(TensorDecl(f"{prefix}{self.names['k_norm']}.weight", (self.hd,), "norm"))
        return out

    def load(self, tensors: Dict[str, torch.Tensor], prefix: str) -> None:
        self.qkv.load(tensors, prefix)
        self.o.load(tensors, prefix)
        if self.qk_norm:
            self.q_norm_w = tensors[f"{prefix}{self.names['q_norm']}.weight"]
            self.k_norm_w = self.q_norm_w if self.shares_cache else tensors[f"{prefix}{self.names['k_norm']}.weight"]
            if self.k_norm_w.dtype != self.q_norm_w.dtype:
                self.q_norm_w, self.k_norm_w = self.q_norm_w.float(), self.k_norm_w.float()

    def weight_bytes(self) -> int:
        return self.qkv.weight_bytes() + self.o.weight_bytes()

    def workspace_bytes(self, n_tokens: int) -> int:
        """Projections, attention output and the delta (as partial sums: up to 8 of each for few tokens)."""
        esz = 4 if self.env.mode == "float32" else 2
        parts = 8 if n_tokens <= 128 else 1
        return n_tokens * (self.qkv.n * max(esz, 4 * parts if parts > 1 else esz) + 2 * self.nq * self.hd * esz
                           + self.hidden * 4 * parts + self.nq * 4 * (self.hd + 2) * (parts if parts > 1 else 0))

    def cost(self, q_lens, kv_lens):
        from ..profile import cost as C
        T = sum(q_lens)
        esz = 4 if self.env.mode == "float32" else 2
        parts = [self.qkv.cost(T), self.o.cost(T),
                 C.attention(q_lens, kv_lens, self.nq, self.nkv, self.hd, esz, int(self.window) if self.window else None)]
        return sum(p[0] for p in parts), sum(p[1] for p in parts)

    can_sink = True        # forward() accepts sink=ResidualSink (see parts.base)

    def takes_deferred(self, batch) -> bool:
        """Whether forward() can be handed a DeferredNorm for this step: the decode kernel that takes
        the projections applies the rows' 1/RMS, which a bias inside the projection would spoil."""
        return (batch.is_decode and self.hd == 128 and not self.bias and self.env.act_dtype == torch.bfloat16
                and self.qkv.weight is not None and self.qkv.weight.dtype == torch.bfloat16
                and self.qkv._splits(batch.n_tokens) > 1
                and (self.shares_cache or self.nq // self.nkv <= 16)     # wider groups: the kernel does not write the cache
                and (self.position.inv_freq is None or self.position.rot_dim == self.hd))

    can_add_into = True    # forward() accepts add_into=residual (see parts.base)

    def forward(self, xn, batch, view, sink=None, add_into=None):
        T = batch.n_tokens
        dev, act = self.env.device, self.env.act_dtype
        qd = self.nq * self.hd
        attn = torch.empty((T, qd), dtype=act, device=dev)
        window = int(self.window) if self.window else 0
        writes = view.writes and not self.shares_cache
        done = False
        if isinstance(xn, DeferredNorm):
            proj = self.qkv.forward_auto(xn.x, T)
            done = self._decode_fused(proj, attn, batch, view, window, writes, xn.rowscale, xn.width)
            if not done:
                xn = xn.materialize()     # the kernel declined after all: the norm's own kernel, then as always
        if not done and not batch.is_decode and self._prompt_fused(xn, attn, batch, view, window, writes):
            done = True
        if not done:
            proj = self.qkv.forward_auto(xn, T)      # [T, N] or [S, T, N] partial sums
            done = batch.is_decode and self._decode_fused(proj, attn, batch, view, window, writes)
        if not done:
            q = proj if proj.dim() == 2 else torch.empty((T, qd), dtype=act, device=dev)
            kernels.qk_norm_rope_cache(
                proj, q, T, self.nq, self.nkv, self.hd, self.q_norm_w, self.k_norm_w, self.qk_norm_eps,
                self.position.inv_freq, self.position.rot_dim, batch.positions, batch.slot_of_token,
                view.block_table, view.k, view.v, write_kv=writes,
                cos_sin=self.position.cos_sin(batch))
            self.attend(q, attn, batch, view, window)
        if sink is not None:
            deferred = self.o.forward_residual(attn, T, sink)
            if deferred is not None:
                return deferred
        if add_into is not None and self.o.forward_add(attn, T, add_into):
            return None
        return self.o.forward_delta(attn, T)

    def _prompt_fused(self, xn, out, batch, view, window, writes) -> bool:
        """Many tokens, head size 128: the projection's own epilogue normalises and rotates the heads
        and writes keys and values into the cache, so the projections never go through memory.
        False: not this time (other sizes, a partial rotation, few tokens)."""
        if self.hd != 128 or self.env.act_dtype != torch.bfloat16 or not isinstance(xn, torch.Tensor) \
                or xn.dtype != torch.bfloat16 or self.qkv.weight is None or self.qkv.weight.dtype != torch.bfloat16:
            return False
        rot = self.position.rot_dim if self.position.inv_freq is not None else 0
        if rot not in (0, self.hd) or writes != (self.qkv.n == (self.nq + 2 * self.nkv) * self.hd):
            return False
        T = batch.n_tokens
        if T < PROMPT_FUSED_MIN_TOKENS:
            return False
        q = torch.empty((T, self.nq * self.hd), dtype=torch.bfloat16, device=xn.device)
        cos_sin = self.position.cos_sin(batch) if rot else None
        with scope(op=self.qkv.label):
            if not kernels.gemm_tcgen05_qkv_rope(
                    xn, self.qkv.weight, q, self.nq, self.nkv, self.q_norm_w, self.k_norm_w, self.qk_norm_eps,
                    cos_sin, batch.positions, batch.slot_of_token,
                    view.block_table, view.k, view.v, self.qkv.bias, T):
                return False
        self.attend(q, out, batch, view, window)
        return True

    def _decode_fused(self, proj, out, batch, view, window, writes, rowscale=None, row_width=0) -> bool:
        """One token per sequence, head size 128, float32 projections: the attention kernel itself
        adds the partial sums, normalises and rotates the queries and writes the new key and value,
        so no kernel stands between the projection and the attention.  False: not this time."""
        if self.hd != 128 or proj.dtype != torch.float32 or view.k.dtype != torch.bfloat16:
            return False
        rot = self.position.rot_dim if self.position.inv_freq is not None else 0
        if rot not in (0, self.hd):
            return False
        n_pages = max(1, (batch.max_kv_len + DECODE_CHUNK - 1) // DECODE_CHUNK)
        groups = self.nkv * ((self.nq // self.nkv + 15) // 16)
        n_blocks, ppb = kernels.decode_split(batch.n_seqs, groups, n_pages, out.device)
        acc = ml = None
        if n_pages > 1:
            T = batch.n_tokens
            parts = max(n_pages, n_blocks)          # the kernel strides a row's partial results by n_blocks
            acc = torch.empty((T, self.nq, parts, self.hd), dtype=torch.float32, device=out.device)
            ml = torch.empty((T, self.nq, parts, 2), dtype=torch.float32, device=out.device)
        return kernels.attention_decode_fused(
            proj, out, view.k, view.v, view.block_table, batch.seq_slot, batch.cu_q, batch.kv_len, batch.n_seqs,
            self.nq, self.nkv, self.hd, self.q_norm_w, self.k_norm_w, self.qk_norm_eps,
            self.position.cos_sin(batch) if rot else None, writes, self.scale, window, n_blocks, acc, ml, ppb,
            rowscale=rowscale, row_width=row_width)

    def attend(self, q, out, batch, view, window):
        """Softmax attention of the step's queries over the cache.  One token per sequence:
        keys split in fixed chunks, partial results merged; otherwise whole rows."""
        if batch.is_decode:
            chunk = DECODE_CHUNK
            T = batch.n_tokens
            n_pages = max(1, (batch.max_kv_len + chunk - 1) // chunk)
            groups = self.nkv * ((self.nq // self.nkv + 15) // 16)
            n_blocks, ppb = kernels.decode_split(batch.n_seqs, groups, n_pages, q.device)
            acc = ml = None
            if n_pages > 1:
                parts = max(n_pages, n_blocks)
                acc = torch.empty((T, self.nq, parts, self.hd), dtype=torch.float32, device=q.device)
                ml = torch.empty((T, self.nq, parts, 2), dtype=torch.float32, device=q.device)
            fast = kernels.attention_decode(q, out, view.k, view.v, view.block_table, batch.seq_slot, batch.cu_q,
                                            batch.kv_len, batch.n_seqs, self.nq, self.nkv, self.hd, self.scale,
                                            window, n_blocks, acc, ml, ppb)
            n_chunks = n_pages
            if fast:
                return
            if n_chunks > 1:
                kernels.attention_generic(q, out, view.k, view.v, view.block_table, batch.seq_slot, batch.cu_q,
                                          batch.kv_len, batch.n_seqs, 1, self.nq, self.nkv, self.hd, self.scale,
                                          window, chunk, n_chunks, acc, ml)
                kernels.attention_merge(acc, ml, out, batch.positions, batch.slot_of_token, T, self.nq, self.hd,
                                        chunk, n_chunks, window)
                return
        if kernels.attention_prefill_tc5(q, batch.n_tokens, out, view.k, view.v, view.block_table, batch.seq_slot,
                                         batch.cu_q, batch.kv_len, batch.n_seqs, batch.max_q_len, self.nq, self.nkv,
                                         self.hd, self.scale, window, max_kv_len=batch.max_kv_len):
            return
        if kernels.attention_prefill(q, out, view.k, view.v, view.block_table, batch.seq_slot, batch.cu_q,
                                     batch.kv_len, batch.n_seqs, batch.max_q_len, self.nq, self.nkv, self.hd,
                                     self.scale, window):
            return
        kernels.attention_generic(q, out, view.k, view.v, view.block_table, batch.seq_slot, batch.cu_q,
                                  batch.kv_len, batch.n_seqs, batch.max_q_len, self.nq, self.nkv, self.hd,
                                  self.scale, window)
