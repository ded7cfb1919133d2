"""A decoder assembled from a ModelSpec: embedding, blocks, the order they run in, final
norm, head.  It is generic: the architecture lives in the spec, not here.

One forward pass (rocml/src/forward/mod.rs:271-378, chunk_forward.rs:97-188): embedding
gather into a 32-bit residual stream; the scheduled blocks; the final norm only on the rows
whose logits are wanted; the head on those rows -> float32 logits.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import kernels
from ..profile import scope
from ..config.specs import MixerSpec, ModelSpec
from ..errors import ConfigError
from ..parts import BuildEnv, build_block, build_norm
from ..parts.linear import Linear
from ..weights.decl import TensorDecl
from ..weights.loader import load_tensors


class Model:
    def __init__(self, spec: ModelSpec, env: BuildEnv):
        self.spec = spec
        self.env = env
        self.hidden = spec.hidden
        self.vocab = spec.vocab
        readers = {e.layer for e in spec.schedule if e.reads_cache_of is not None}
        owners = {e.layer for e in spec.schedule if e.reads_cache_of is None}
        if readers & owners:
            raise ConfigError("a layer cannot both keep its own cache and read another's in one schedule")
        self.blocks = []
        for i, layer in enumerate(spec.layers):
            mixer_spec = layer.mixer
            if i in readers:
                mixer_spec = MixerSpec(mixer_spec.kind, tuple(sorted({**mixer_spec.params, "shares_cache": True}.items())),
                                       mixer_spec.position)
            self.blocks.append(build_block_with(layer, spec.hidden, env, mixer_spec))
        self.final_norm = build_norm(spec.final_norm, spec.hidden, env)
        self.head = Linear([spec.head_name[: -len(".weight")]], [spec.vocab], spec.hidden, False, env)
        self.embed: Optional[torch.Tensor] = None
        self.status: Optional[torch.Tensor] = None

    # ---- tensors ------------------------------------------------------------------------------
    def declare(self) -> List[TensorDecl]:
        out = [TensorDecl(self.spec.embedding_name, (self.vocab, self.hidden), "matrix")]
        for b in self.blocks:
            out += b.declare()
        out += self.final_norm.declare(self.spec.final_norm_name[: -len(".weight")])
        if not self.spec.tie_embeddings:
            out += self.head.declare("")
        return out

    def ignorable(self) -> List[str]:
        """Tensors a folder may hold that the model does not read: a stored head when the
        head is tied to the embedding."""
        return [self.spec.head_name] if self.spec.tie_embeddings else []

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.embed = tensors[self.spec.embedding_name]
        for b in self.blocks:
            b.load(tensors)
        self.final_norm.load(tensors, self.spec.final_norm_name[: -len(".weight")])
        if self.spec.tie_embeddings:
            self.head.adopt(self.embed)
        else:
            self.head.load(tensors, "")
        self.status = torch.zeros(1, dtype=torch.int32, device=self.env.device)

    def load_folder(self, folder: str) -> None:
        self.load(load_tensors(folder, self.declare(), self.env.mode, self.env.device, self.ignorable()))

    def load_random(self, seed: int) -> None:
        """Random weights made directly on the device (the distributions of the random-weights
        mode; no folder is written)."""
        from ..weights.random_init import random_tensor
        dt = torch.float32 if self.env.mode == "float32" else torch.bfloat16
        tensors = {}
        for d in self.declare():
            t = random_tensor(d, seed, self.env.device, torch.bfloat16)
            tensors[d.name] = t if d.role == "int_table" else t.to(dt)
        self.load(tensors)

    # ---- facts ----------------------------------------------------------------------------------
    @property
    def graph_safe(self) -> bool:
        return all(b.graph_safe for b in self.blocks) and self.final_norm.graph_safe

    def cache_requirements(self):
        return [self.blocks[e.layer].mixer.cache_requirement() for e in self.spec.schedule]

    def reads_cache_of(self):
        return [e.reads_cache_of for e in self.spec.schedule]

    def weight_bytes_per_step(self) -> int:
        """Bytes of weights a step reads once: every scheduled block, the final norm, the head
        (the embedding rows it gathers are negligible)."""
        n = sum(self.blocks[e.layer].weight_bytes() for e in self.spec.schedule)
        return n + self.final_norm.weight_bytes() + self.head.weight_bytes()

    def workspace_bytes(self, n_tokens: int, n_want: int) -> int:
        """Device memory a step of ``n_tokens`` tokens allocates besides weights and cache: the 32-bit
        residual stream, the widest layer's buffers (asked of the parts: layers run one after another,
        and a delta outlives its layer by one norm), and float32 logits for ``n_want`` rows."""
        widest = max([getattr(b, "workspace_bytes", lambda n: 0)(n_tokens) for b in self.blocks] or [0])
        return n_tokens * self.hidden * 4 * 2 + 2 * widest + n_want * (self.vocab * 4 + self.hidden * 4)

    def step_cost(self, q_lens, kv_lens, n_want: int):
        """(bytes, floating-point operations) a step has to move and do at least: every scheduled
        block's weights once and its products and attention over the given sequences (``q_lens`` new
        tokens each, ``kv_lens`` long afterwards, whose keys and values are read once), the final norm,
        and the head on ``n_want`` rows.  Asked of the parts, so it holds for any arrangement."""
        nbytes = flops = 0
        for e in self.spec.schedule:
            block = self.blocks[e.layer]
            if hasattr(block, "cost"):
                b, f = block.cost(q_lens, kv_lens)
            else:
                b, f = block.weight_bytes(), 0
            nbytes, flops = nbytes + b, flops + f
        hb, hf = self.head.cost(n_want)
        return nbytes + self.final_norm.weight_bytes() + hb, flops + hf

    # ---- the pass ---------------------------------------------------------------------------------
    def forward(self, batch, cache) -> Optional[torch.Tensor]:
        T = batch.n_tokens
        resid = torch.empty((T, self.hidden), dtype=torch.float32, device=self.env.device)
        with scope(op="embedding"):
            kernels.embedding(batch.token_ids, self.embed, resid, self.status)
        pending = None
        sched = self.spec.schedule
        for i, e in enumerate(sched):
            block = self.blocks[e.layer]
            with scope(layer=i):
                if getattr(block, "chains", False):
                    # a block may prepare the first norm of the block that follows it
                    nxt = self.blocks[sched[i + 1].layer] if i + 1 < len(sched) else None
                    pending = block.forward(resid, pending, batch, cache.views[i], next_block=nxt)
                else:
                    pending = block.forward(resid, pending, batch, cache.views[i])
        if batch.n_want == 0:
            return None
        with scope(op="final_norm"):
            xn = self.final_norm.forward(resid, pending, n_rows=batch.n_want, rows=batch.want_rows, write_back=False)
        logits = torch.empty((batch.n_want, self.vocab), dtype=torch.float32, device=self.env.device)
        self.head.forward(xn, logits, batch.n_want)
        return logits


def build_block_with(layer, hidden, env, mixer_spec):
    from ..parts.base import _lookup, _ARRANGEMENTS
    return _lookup(_ARRANGEMENTS, layer.arrangement, "arrangement")(layer, hidden, env, mixer_spec)


def declared_tensors(spec: ModelSpec) -> List[TensorDecl]:
    """The tensors a model of this spec reads from its folder (no device memory is touched)."""
    return Model(spec, BuildEnv(torch.device("cpu"), torch.bfloat16)).declare()
